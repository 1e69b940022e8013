// SSD chunk outputs on the 5th-generation tensor cores (tcgen05 + TMEM), for the Mamba-2 / Mamba-3 paths:
//     y[t, h, :] = sum_{s <= t, same chunk} exp(cum_h[t] - cum_h[s]) (C_t . B_s) xw[s, h, :]      (intra-chunk)
//                + exp(cum_h[t]) C_t . prev_h                                                     (state entering the chunk)
// with chunk 64, head dim 64, state dim 128 (cum = inclusive cumulative sum of log a inside the chunk).
//
// One CTA owns two consecutive chunks of one sequence = 128 time steps = the 128 TMEM lanes of an M = 128 MMA:
//   G  = [C_c; C_c+1] . [B_c; B_c+1]^T   128 x 128, K = 128, ONCE for all heads (B and C are shared by the heads)
// and then per head
//   M_h = G masked to the two causal 64 x 64 diagonal blocks and scaled by the decay: written by the epilogue
//         threads as bf16 into shared memory in the K-major swizzled layout an A operand has,
//   Y1 = M_h . xw_h                       128 x 64, K = 128 (the off-diagonal blocks are zeros)
//   Y2 = [C_c; C_c+1] . prev_h(chunk c) and . prev_h(chunk c+1)    two 128 x 64 products, K = 128; rows 0-63 are
//         taken from the first, rows 64-127 from the second,
//   y  = Y1 + exp(cum) * Y2.
// Operands are rounded to bf16 (fp32 accumulation in TMEM), as in the other GEMMs of this library; the fp32 FMA
// kernels of ssd.cu stay as the exact path. The per-chunk states come from ssd.cu's state kernels. The reference has
// no Mamba path; the algorithm is Mamba-2's SSD (Dao & Gu, 2024).
#include "bdh_kernels.h"
#include "device_once.h"
#include "sm100_ptx.cuh"

namespace bdh {

constexpr int TC_Q = 64, TC_P = 64, TC_N = 128, TC_ROWS = 128, TC_THREADS = 256;
constexpr int TC_TILE = TC_ROWS * 128 * 2;        // [128 x 128] bf16, two [128 x 64] K-major boxes: 32 KB
constexpr int TC_BTILE = 128 * TC_P * 2;          // [128 k x 64] bf16 MN-major: 16 KB

struct SsdTcSmem {
  static constexpr int C2 = 0;
  static constexpr int B2 = C2 + TC_TILE;
  static constexpr int MH = B2 + TC_TILE;
  static constexpr int XH = MH + TC_TILE;
  static constexpr int H0 = XH + TC_BTILE;
  static constexpr int H1 = H0 + TC_BTILE;
  static constexpr int CUM = H1 + TC_BTILE;       // [128] fp32
  static constexpr int BAR = CUM + 512;
  static constexpr int TOTAL = BAR + 64 + 1024;
};

// element (row, k) of a K-major [128 x 128] bf16 tile: box k / 64, 128-byte rows, 16-byte chunks XOR-swizzled by row
__device__ __forceinline__ uint32_t kmajor_off(int row, int k) {
  return static_cast<uint32_t>((k >> 6) * (TC_ROWS * 128) + row * 128 + ((((k & 63) >> 3) ^ (row & 7)) << 4) + (k & 7) * 2);
}
// element (k, n) of an MN-major [128 k x 64 n] bf16 operand (rows are k): 128-byte rows, swizzled by k
__device__ __forceinline__ uint32_t mnmajor_off(int k, int n) {
  return static_cast<uint32_t>(k * 128 + (((n >> 3) ^ (k & 7)) << 4) + (n & 7) * 2);
}

// fp32 [rows_valid x 128] (row pitch 128) -> K-major bf16 tile; rows beyond rows_valid are zero
__device__ __forceinline__ void load_kmajor_128(uint8_t* tile, const float* src, int rows_valid) {
  for (int i = threadIdx.x; i < TC_ROWS * 16; i += TC_THREADS) {      // 16 chunks of 8 columns per row
    const int row = i >> 4, k0 = (i & 15) * 8;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows_valid) {
      const float4 a = *reinterpret_cast<const float4*>(src + static_cast<long long>(row) * 128 + k0);
      const float4 b = *reinterpret_cast<const float4*>(src + static_cast<long long>(row) * 128 + k0 + 4);
      u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w);
      u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
    }
    *reinterpret_cast<uint4*>(tile + kmajor_off(row, k0)) = u;
  }
}

// fp32 [rows_valid x 64] with row pitch `pitch` floats -> MN-major bf16 operand [128 k x 64]; rows beyond are zero
__device__ __forceinline__ void load_mnmajor_64(uint8_t* tile, const float* src, long long pitch, int rows_valid) {
  for (int i = threadIdx.x; i < 128 * 8; i += TC_THREADS) {           // 8 chunks of 8 columns per row
    const int k = i >> 3, n0 = (i & 7) * 8;
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (k < rows_valid) {
      const float4 a = *reinterpret_cast<const float4*>(src + k * pitch + n0);
      const float4 b = *reinterpret_cast<const float4*>(src + k * pitch + n0 + 4);
      u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w);
      u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
    }
    *reinterpret_cast<uint4*>(tile + mnmajor_off(k, n0)) = u;
  }
}

// xw [B,T,H,64], loga [B,T,H], Bm/Cm [B,T,128], states [B,C,H,128,64] = state ENTERING each chunk, y [B,T,H,64].
__global__ void __launch_bounds__(TC_THREADS, 1)
ssd_chunk_out_tc_kernel(const float* __restrict__ xw, const float* __restrict__ loga, const float* __restrict__ Bm,
                        const float* __restrict__ Cm, const float* __restrict__ states, float* __restrict__ y, int T,
                        int H, int C, int* status) {
  using L = SsdTcSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  float* cum = reinterpret_cast<float*>(smem + L::CUM);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x, b = blockIdx.y;
  const int c0 = pair * 2;
  const int rows_valid = (c0 + 1 < C) ? TC_ROWS : TC_Q;       // an odd chunk count leaves the last CTA half full
  const long long t0 = static_cast<long long>(b) * T + static_cast<long long>(c0) * TC_Q;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_G = 0, COL_Y1 = 128, COL_Y2A = 192, COL_Y2B = 256;

  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  load_kmajor_128(smem + L::C2, Cm + t0 * TC_N, rows_valid);
  load_kmajor_128(smem + L::B2, Bm + t0 * TC_N, rows_valid);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  uint32_t phase = 0;
  bool ok = true;

  // ---- G = C2 . B2^T ----
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t sa = smem_u32(smem + L::C2), sb = smem_u32(smem + L::B2);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t off = (k >> 2) * (TC_ROWS * 128) + (k & 3) * 32;
      umma_bf16(tmem_base + COL_G, make_smem_desc(sa + off, 16, 1024), make_smem_desc(sb + off, 16, 1024), idesc,
                k > 0 ? 1u : 0u);
    }
    umma_commit(bar);
  }
  ok = mbar_wait(bar, phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
  phase ^= 1;
  tc_fence_after();

  const int q = warp & 3;                      // TMEM lane quarter of this warp (warps 0-3 are the epilogue warps)
  const int row = q * 32 + lane;               // time step inside the pair of chunks (epilogue threads)
  const int chunk_of_row = row >> 6;
  for (int h = 0; h < H && ok; ++h) {
    // ---- per-head operands: cumulative log-decay, xw_h, the two entering states ----
    if (warp == 4) {
      // two independent inclusive scans of 64 steps (one per chunk): lane l holds steps 2l and 2l+1 of each
      for (int cc = 0; cc < 2; ++cc) {
        float a0 = 0.f, a1 = 0.f;
        if (cc * TC_Q < rows_valid) {
          a0 = loga[(t0 + cc * TC_Q + 2 * lane) * H + h];
          a1 = loga[(t0 + cc * TC_Q + 2 * lane + 1) * H + h];
        }
        float s = a0 + a1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float o = __shfl_up_sync(0xffffffffu, s, d);
          if (lane >= d) s += o;
        }
        cum[cc * TC_Q + 2 * lane] = s - a1;
        cum[cc * TC_Q + 2 * lane + 1] = s;
      }
    }
    load_mnmajor_64(smem + L::XH, xw + (t0 * H + h) * TC_P, static_cast<long long>(H) * TC_P, rows_valid);
    const float* st0 = states + ((static_cast<long long>(b) * C + c0) * H + h) * TC_N * TC_P;
    load_mnmajor_64(smem + L::H0, st0, TC_P, TC_N);
    load_mnmajor_64(smem + L::H1, st0 + static_cast<long long>(H) * TC_N * TC_P, TC_P, rows_valid > TC_Q ? TC_N : 0);
    __syncthreads();
    // ---- M_h: masked, decayed scores as the A operand of the next product ----
    if (warp < 4) {
      const float cr = cum[row];
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        float v[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + COL_G + cb * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float w[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int s = cb * 32 + j * 8 + e;
            const bool on = ((s >> 6) == chunk_of_row) && (s <= row);
            w[e] = on ? v[j * 8 + e] * __expf(cr - cum[s]) : 0.f;
          }
          uint4 u;
          u.x = pack_bf16x2(w[0], w[1]); u.y = pack_bf16x2(w[2], w[3]);
          u.z = pack_bf16x2(w[4], w[5]); u.w = pack_bf16x2(w[6], w[7]);
          *reinterpret_cast<uint4*>(smem + L::MH + kmajor_off(row, cb * 32 + j * 8)) = u;
        }
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // ---- Y1 = M_h . xw_h ; Y2a = C2 . prev(c) ; Y2b = C2 . prev(c+1) ----
    if (threadIdx.x == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 64, 0, 1);
      const uint32_t sm_ = smem_u32(smem + L::MH), sc = smem_u32(smem + L::C2);
      const uint32_t sx = smem_u32(smem + L::XH), s0 = smem_u32(smem + L::H0), s1 = smem_u32(smem + L::H1);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t aoff = (k >> 2) * (TC_ROWS * 128) + (k & 3) * 32;
        const uint32_t boff = k * 2048;          // 16 k-rows of 128 bytes
        umma_bf16(tmem_base + COL_Y1, make_smem_desc(sm_ + aoff, 16, 1024), make_smem_desc(sx + boff, 8192, 1024), idesc,
                  k > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t aoff = (k >> 2) * (TC_ROWS * 128) + (k & 3) * 32;
        const uint32_t boff = k * 2048;
        umma_bf16(tmem_base + COL_Y2A, make_smem_desc(sc + aoff, 16, 1024), make_smem_desc(s0 + boff, 8192, 1024), idesc,
                  k > 0 ? 1u : 0u);
        umma_bf16(tmem_base + COL_Y2B, make_smem_desc(sc + aoff, 16, 1024), make_smem_desc(s1 + boff, 8192, 1024), idesc,
                  k > 0 ? 1u : 0u);
      }
      umma_commit(bar);
    }
    ok = mbar_wait(bar, phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
    phase ^= 1;
    tc_fence_after();
    // ---- y = Y1 + exp(cum) * Y2 ----
    if (warp < 4 && ok && row < rows_valid) {
      const float w = __expf(cum[row]);
      const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      float* out = y + ((t0 + row) * H + h) * TC_P;
#pragma unroll 1
      for (int cb = 0; cb < 2; ++cb) {
        float v1[32], v2[32];
        tmem_ld_32x32(lane_base + COL_Y1 + cb * 32, v1);
        tmem_ld_32x32(lane_base + (chunk_of_row ? COL_Y2B : COL_Y2A) + cb * 32, v2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(out + cb * 32 + 4 * j) =
              make_float4(v1[4 * j] + w * v2[4 * j], v1[4 * j + 1] + w * v2[4 * j + 1], v1[4 * j + 2] + w * v2[4 * j + 2],
                          v1[4 * j + 3] + w * v2[4 * j + 3]);
      }
    }
    tc_fence_before();
    __syncthreads();          // the next head overwrites the operands, the scores tile and the accumulators
    tc_fence_after();
  }
  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace bdh

using namespace bdh;

// Same contract as bdh_ssd_chunk_scan, with the chunk outputs computed on the tensor cores (bf16 operands,
// fp32 accumulation); the per-chunk states and the pass over the chunks are the fp32 kernels of ssd.cu.
extern "C" int bdh_ssd_chunk_scan_tc(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                                     float* states, float* decay, float* y, int B, int T, int H, int* status,
                                     cudaStream_t s) {
  if (B <= 0 || H <= 0 || T <= 0 || (T % TC_Q)) return BDH_ERR_ARGUMENT;
  for (const void* p : {static_cast<const void*>(xw), static_cast<const void*>(Bm), static_cast<const void*>(Cm),
                        static_cast<const void*>(states), static_cast<const void*>(y)})
    if (reinterpret_cast<uintptr_t>(p) & 15) return BDH_ERR_ALIGNMENT;
  int rc = bdh_ssd_chunk_states(xw, loga, Bm, h, states, decay, B, T, H, s);
  if (rc != BDH_OK) return rc;
  const int C = T / TC_Q;
  static PerDeviceOnce configured;
  if (configured.run([&] {
        return cudaFuncSetAttribute(ssd_chunk_out_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SsdTcSmem::TOTAL) == cudaSuccess ? 0 : 1;
      }))
    return BDH_ERR_LAUNCH;
  dim3 grid((C + 1) / 2, B);
  ssd_chunk_out_tc_kernel<<<grid, TC_THREADS, SsdTcSmem::TOTAL, s>>>(xw, loga, Bm, Cm, states, y, T, H, C, status);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}
