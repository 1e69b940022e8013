// Chunked SSD scan for the Mamba-2 / Mamba-3 paths (chunk 64, head dim 64, state dim 128, fp32):
//     h_t = exp(loga_t) h_{t-1} + B_t (x) xw_t ;  y_t = C_t . h_t
// Three launches: per-chunk states, a pass over the chunks that turns them into the state entering
// each chunk (and the final state), then the per-chunk outputs (intra-chunk quadratic part plus the
// carried state). `states` [B, C, H, N, P] is scratch owned by the caller. The reference has no
// Mamba path; the algorithm is Mamba-2's SSD (Dao & Gu, 2024).
#include "bdh_kernels.h"
#include "device_once.h"

namespace bdh {

constexpr int SSD_Q = 64, SSD_P = 64, SSD_N = 128, SSD_THREADS = 256;

// inclusive cumulative sum of loga over the chunk, in shared memory (thread 0..63 hold one step)
__device__ __forceinline__ void chunk_cumsum(const float* loga, long long stride, float* cum) {
  if (threadIdx.x < SSD_Q) cum[threadIdx.x] = loga[threadIdx.x * stride];
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < SSD_Q; ++i) { s += cum[i]; cum[i] = s; }
  }
  __syncthreads();
}

// xw [B,T,H,P], loga [B,T,H], Bm [B,T,N] -> states[b,c,h,n,p] = sum_j exp(cum_last - cum_j) B[j,n] xw[j,p]
__global__ void __launch_bounds__(SSD_THREADS)
ssd_chunk_state_kernel(const float* __restrict__ xw, const float* __restrict__ loga, const float* __restrict__ Bm,
                       float* __restrict__ states, float* __restrict__ chunk_decay, int T, int H) {
  extern __shared__ float sm[];
  float* sx = sm;                          // [Q][P]  (pre-multiplied by the decay to the chunk end)
  float* sb = sx + SSD_Q * SSD_P;          // [Q][N]
  float* cum = sb + SSD_Q * SSD_N;         // [Q]
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, C = gridDim.x;
  const long long t0 = static_cast<long long>(b) * T + static_cast<long long>(c) * SSD_Q;
  chunk_cumsum(loga + t0 * H + h, H, cum);
  const float last = cum[SSD_Q - 1];
  for (int i = threadIdx.x; i < SSD_Q * SSD_P; i += SSD_THREADS) {
    int j = i / SSD_P, p = i % SSD_P;
    sx[i] = xw[((t0 + j) * H + h) * SSD_P + p] * __expf(last - cum[j]);
  }
  for (int i = threadIdx.x; i < SSD_Q * SSD_N; i += SSD_THREADS) sb[i] = Bm[t0 * SSD_N + i];
  __syncthreads();
  // 128 x 64 outputs, 256 threads: thread owns a 4 (n) x 8 (p) tile
  const int tn = (threadIdx.x / 8) * 4, tp = (threadIdx.x % 8) * 8;
  float acc[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[a][q] = 0.f;
  for (int j = 0; j < SSD_Q; ++j) {
    float bv[4], xv[8];
#pragma unroll
    for (int a = 0; a < 4; ++a) bv[a] = sb[j * SSD_N + tn + a];
#pragma unroll
    for (int q = 0; q < 8; ++q) xv[q] = sx[j * SSD_P + tp + q];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[a][q] += bv[a] * xv[q];
  }
  float* out = states + ((static_cast<long long>(b) * C + c) * H + h) * SSD_N * SSD_P;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int q = 0; q < 8; ++q) out[(tn + a) * SSD_P + tp + q] = acc[a][q];
  if (threadIdx.x == 0) chunk_decay[(static_cast<long long>(b) * C + c) * H + h] = __expf(last);
}

// In place: states[b,c,h] <- state entering chunk c ; h <- state after the last chunk.
__global__ void ssd_state_pass_kernel(float* __restrict__ states, const float* __restrict__ chunk_decay,
                                      float* __restrict__ h, int C, int H, long long total /* B*H*N*P */) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long np = SSD_N * SSD_P;
  const long long bh = i / np, e = i % np;
  const long long b = bh / H, hh = bh % H;
  float cur = h[i];
  for (int c = 0; c < C; ++c) {
    const long long idx = ((b * C + c) * H + hh) * np + e;
    const float s = states[idx];
    states[idx] = cur;
    cur = cur * chunk_decay[(b * C + c) * H + hh] + s;
  }
  h[i] = cur;
}

// y[i,p] = sum_{j<=i} exp(cum_i - cum_j) (C_i . B_j) xw[j,p] + exp(cum_i) sum_n C[i,n] prev[n,p]
__global__ void __launch_bounds__(SSD_THREADS)
ssd_chunk_out_kernel(const float* __restrict__ xw, const float* __restrict__ loga, const float* __restrict__ Bm,
                     const float* __restrict__ Cm, const float* __restrict__ states, float* __restrict__ y, int T,
                     int H) {
  extern __shared__ float sm[];
  float* sx = sm;                           // [Q][P]
  float* sb = sx + SSD_Q * SSD_P;           // [Q][N]
  float* sc = sb + SSD_Q * SSD_N;           // [Q][N]
  float* sp = sc + SSD_Q * SSD_N;           // [N][P]  state entering the chunk
  float* sl = sp + SSD_N * SSD_P;           // [Q][Q]  masked decay * (C B^T)
  float* cum = sl + SSD_Q * SSD_Q;          // [Q]
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z, C = gridDim.x;
  const long long t0 = static_cast<long long>(b) * T + static_cast<long long>(c) * SSD_Q;
  chunk_cumsum(loga + t0 * H + h, H, cum);
  for (int i = threadIdx.x; i < SSD_Q * SSD_P; i += SSD_THREADS) {
    int j = i / SSD_P, p = i % SSD_P;
    sx[i] = xw[((t0 + j) * H + h) * SSD_P + p];
  }
  for (int i = threadIdx.x; i < SSD_Q * SSD_N; i += SSD_THREADS) {
    sb[i] = Bm[t0 * SSD_N + i];
    sc[i] = Cm[t0 * SSD_N + i];
  }
  const float* prev = states + ((static_cast<long long>(b) * C + c) * H + h) * SSD_N * SSD_P;
  for (int i = threadIdx.x; i < SSD_N * SSD_P; i += SSD_THREADS) sp[i] = prev[i];
  __syncthreads();
  // scores: 64 x 64, thread owns a 4 x 4 tile
  const int ti = (threadIdx.x / 16) * 4, tj = (threadIdx.x % 16) * 4;
  {
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[a][q] = 0.f;
    for (int n = 0; n < SSD_N; ++n) {
      float cv[4], bv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) { cv[a] = sc[(ti + a) * SSD_N + n]; bv[a] = sb[(tj + a) * SSD_N + n]; }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[a][q] += cv[a] * bv[q];
    }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = ti + a, j = tj + q;
        sl[i * SSD_Q + j] = (j <= i) ? acc[a][q] * __expf(cum[i] - cum[j]) : 0.f;
      }
  }
  __syncthreads();
  // outputs: 64 x 64, thread owns rows ti..ti+3, columns tp..tp+3
  const int tp = tj;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[a][q] = 0.f;
  for (int j = 0; j < SSD_Q; ++j) {
    float lv[4], xv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) { lv[a] = sl[(ti + a) * SSD_Q + j]; xv[a] = sx[j * SSD_P + tp + a]; }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[a][q] += lv[a] * xv[q];
  }
  float carry[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int q = 0; q < 4; ++q) carry[a][q] = 0.f;
  for (int n = 0; n < SSD_N; ++n) {
    float cv[4], pv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) { cv[a] = sc[(ti + a) * SSD_N + n]; pv[a] = sp[n * SSD_P + tp + a]; }
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int q = 0; q < 4; ++q) carry[a][q] += cv[a] * pv[q];
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const float w = __expf(cum[ti + a]);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      y[((t0 + ti + a) * H + h) * SSD_P + tp + q] = acc[a][q] + w * carry[a][q];
  }
}

// One decode step for every (stream, head): h <- exp(loga) h + B (x) xw ; y = C . h. The state is read and
// written once (the torch statement of the step makes four passes over it and materialises the outer product).
// Grid (H, B), 256 threads: thread (g, p) walks 32 of the 128 state rows for column p.
__global__ void __launch_bounds__(256)
ssd_decode_step_kernel(const float* __restrict__ xw, const float* __restrict__ loga, const float* __restrict__ Bm,
                       const float* __restrict__ Cm, float* __restrict__ h, float* __restrict__ y, int H) {
  const int hh = blockIdx.x, b = blockIdx.y;
  const int p = threadIdx.x & 63, g = threadIdx.x >> 6;
  __shared__ float sb[SSD_N], sc[SSD_N], red[4][SSD_P];
  if (threadIdx.x < SSD_N) {
    sb[threadIdx.x] = Bm[static_cast<long long>(b) * SSD_N + threadIdx.x];
    sc[threadIdx.x] = Cm[static_cast<long long>(b) * SSD_N + threadIdx.x];
  }
  __syncthreads();
  const long long bh = static_cast<long long>(b) * H + hh;
  const float a = __expf(loga[bh]);
  const float x = xw[bh * SSD_P + p];
  float* st = h + bh * SSD_N * SSD_P + p;
  float acc = 0.f;
  float v[8];
#pragma unroll 1
  for (int n0 = g * 32; n0 < g * 32 + 32; n0 += 8) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __ldcs(st + (n0 + i) * SSD_P);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = a * v[i] + sb[n0 + i] * x;
      acc += sc[n0 + i] * v[i];
      __stcs(st + (n0 + i) * SSD_P, v[i]);
    }
  }
  red[g][p] = acc;
  __syncthreads();
  if (g == 0) y[bh * SSD_P + p] = red[0][p] + red[1][p] + red[2][p] + red[3][p];
}

}  // namespace bdh

using namespace bdh;

// xw [B,H,64], loga [B,H], Bm/Cm [B,128], h [B,H,128,64] updated in place, y [B,H,64].
extern "C" int bdh_ssd_decode_step(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                                   float* y, int B, int H, cudaStream_t s) {
  if (B <= 0 || H <= 0) return BDH_ERR_ARGUMENT;
  ssd_decode_step_kernel<<<dim3(H, B), 256, 0, s>>>(xw, loga, Bm, Cm, h, y, H);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// xw [B,T,H,64], loga [B,T,H], Bm/Cm [B,T,128], h [B,H,128,64] in/out, states [B,T/64,H,128,64] scratch,
// decay [B,T/64,H] scratch, y [B,T,H,64]; T % 64 == 0.
// First two launches of the scan: per-chunk states and the pass over the chunks. Afterwards states[b,c,h] is the
// state ENTERING chunk c and h the state after the last chunk.
extern "C" int bdh_ssd_chunk_states(const float* xw, const float* loga, const float* Bm, float* h, float* states,
                                    float* decay, int B, int T, int H, cudaStream_t s) {
  if (B <= 0 || H <= 0 || T <= 0 || (T % SSD_Q)) return BDH_ERR_ARGUMENT;
  const int C = T / SSD_Q;
  dim3 grid(C, H, B);
  const int smem_a = (SSD_Q * SSD_P + SSD_Q * SSD_N + SSD_Q) * 4;
  static PerDeviceOnce configured;   // the shared-memory limit is a per-device attribute
  if (configured.run([&] {
        return cudaFuncSetAttribute(ssd_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_a) == cudaSuccess
                   ? 0 : 1;
      }))
    return BDH_ERR_LAUNCH;
  ssd_chunk_state_kernel<<<grid, SSD_THREADS, smem_a, s>>>(xw, loga, Bm, states, decay, T, H);
  const long long total = static_cast<long long>(B) * H * SSD_N * SSD_P;
  ssd_state_pass_kernel<<<static_cast<int>((total + 255) / 256), 256, 0, s>>>(states, decay, h, C, H, total);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_ssd_chunk_scan(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                                  float* states, float* decay, float* y, int B, int T, int H, cudaStream_t s) {
  int rc = bdh_ssd_chunk_states(xw, loga, Bm, h, states, decay, B, T, H, s);
  if (rc != BDH_OK) return rc;
  const int C = T / SSD_Q;
  dim3 grid(C, H, B);
  const int smem_c = (SSD_Q * SSD_P + 2 * SSD_Q * SSD_N + SSD_N * SSD_P + SSD_Q * SSD_Q + SSD_Q) * 4;
  static PerDeviceOnce configured;
  if (configured.run([&] {
        return cudaFuncSetAttribute(ssd_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_c) == cudaSuccess
                   ? 0 : 1;
      }))
    return BDH_ERR_LAUNCH;
  ssd_chunk_out_kernel<<<grid, SSD_THREADS, smem_c, s>>>(xw, loga, Bm, Cm, states, y, T, H);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant: the per-chunk scratch is a fixed array owned by the library.
// ------------------------------------------------------------------------------------------------
#include "bdh_static_scratch.h"

#include <mutex>
#include <stdio.h>

namespace {

constexpr long long STATIC_STATE_FLOATS =
    static_cast<long long>(BDH_SSD_STATIC_MAX_CHUNK_HEADS) * bdh::SSD_N * bdh::SSD_P;
constexpr long long STATIC_TOTAL_FLOATS = STATIC_STATE_FLOATS + BDH_SSD_STATIC_MAX_CHUNK_HEADS;

// In host code this name is only a handle for the runtime; its device address is obtained below.
static __device__ __align__(256) float g_ssd_static_scratch[STATIC_TOTAL_FLOATS];

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mutex;
float* g_static_ptr[MAX_DEVICES] = {};

// Device address of the scratch array on the current device, resolved once per device.
int static_scratch_ptr(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return BDH_ERR_ARGUMENT;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    cudaError_t rc = cudaGetSymbolAddress(&p, g_ssd_static_scratch);
    if (rc != cudaSuccess || !p) {
      fprintf(stderr, "bdh_ssd_chunk_scan_static: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(rc));
      return BDH_ERR_DRIVER;
    }
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return BDH_OK;
}

}  // namespace

extern "C" int bdh_ssd_chunk_scan_static(const float* xw, const float* loga, const float* Bm, const float* Cm,
                                         float* h, float* y, int B, int T, int H, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || T <= 0 || (T % bdh::SSD_Q)) return BDH_ERR_ARGUMENT;
  const long long chunk_heads = static_cast<long long>(B) * (T / bdh::SSD_Q) * H;
  if (chunk_heads > BDH_SSD_STATIC_MAX_CHUNK_HEADS) {
    fprintf(stderr,
            "bdh_ssd_chunk_scan_static: B*(T/64)*H = %lld exceeds the built-in scratch for %d chunk-heads; "
            "use bdh_ssd_chunk_scan with caller-provided scratch\n",
            chunk_heads, BDH_SSD_STATIC_MAX_CHUNK_HEADS);
    return BDH_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != BDH_OK) return rc;
  float* states = scratch;                          // [B, T/64, H, 128, 64]
  float* decay = scratch + STATIC_STATE_FLOATS;     // [B, T/64, H]
  return bdh_ssd_chunk_scan(xw, loga, Bm, Cm, h, states, decay, y, B, T, H, stream);
}
