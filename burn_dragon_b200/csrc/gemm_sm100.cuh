// Persistent, warp-specialised bf16 GEMM for sm_100a with fused epilogues.
//
//   C[z][m, n] = epilogue( sum_k A[z][m, k] * B[z][n, k] )
//
// One CTA per SM loops over output tiles (128 x BN). Warp 0 feeds a ring of shared-memory
// stages with TMA, warp 1 issues tcgen05.mma into one of two TMEM accumulators, warps 2-5 read
// the finished accumulator back with tcgen05.ld and run the epilogue while the MMA warp already
// works on the next tile. Operands may be K-major (rows index m/n, columns index k) or MN-major
// (rows index k, columns index m/n), so activations and weights are consumed in the layout they
// already have, including the transposed products of the backward pass.
//
// The epilogues are the BDH layer's elementwise stages (reference: src/model/bdh.rs:337-441,
// src/kernel/relu_lowrank.rs:7-37, src/model/attention.rs:305-349): ReLU sparsifier with the
// rotary rotation, the x*y gate, the causal decay mask of linear attention, and their backward
// counterparts, so the big [tokens, neurons] tensors cross HBM once per GEMM.
#pragma once
#include "sm100_ptx.cuh"

namespace bdh {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_EPI_WARPS = 4;
constexpr int GEMM_THREADS = 32 * (2 + GEMM_EPI_WARPS);

enum EpiKind : int {
  EPI_STORE = 0,       // out0 = alpha*acc (+ beta*out0); bf16 or fp32 by flag
  EPI_RELU = 1,        // x = relu(acc - theta) -> out0 ; optional q = rot(x) -> out1
  EPI_RELU_GATE = 2,   // y = relu(acc - theta) -> out0 (optional) ; xy = y * in0 -> out1
  EPI_CAUSAL = 3,      // out0 = mask(t, s) * acc * exp(-slope*|t-s|)
  EPI_GATE_BWD = 4,    // g = acc ; out0 = g*in0*(in1>0) ; out1 = g*in1
  EPI_DQ_BWD = 5,      // dq = rot^-1(acc) ; out0 = (dq + in1) * (in0 > 0)
};

enum EpiFlags : int {
  EPI_F_OUT_F32 = 1,       // EPI_STORE: out0 is fp32 (else bf16)
  EPI_F_ACCUM = 2,         // EPI_STORE: out0 += (beta = 1)
  EPI_F_ROPE = 4,          // EPI_RELU: also write the RoPE-rotated copy to out1; EPI_DQ_BWD: undo it
  EPI_F_POPE = 8,          // EPI_RELU: write softplus(x)*[cos, sin] to out1 (real | imag halves)
  EPI_F_UPPER = 16,        // EPI_CAUSAL: write only s > t (else: write everything, zero where s >= t)
  EPI_F_NO_OUT0 = 32,      // EPI_RELU_GATE: skip storing y
  EPI_F_HAS_IN1 = 64,      // EPI_DQ_BWD: add in1
};

struct OperandOffsets {
  long long mn0, mn1;  // element offsets along the m/n dimension per unit of z0, z1
  long long k0, k1;    // element offsets along k per unit of z0, z1
};

struct EpiParams {
  void* out0;
  void* out1;
  const void* in0;
  const void* in1;
  long long ld_out0, ld_out1, ld_in0, ld_in1;
  long long c_m0, c_m1, c_n0, c_n1;      // C row / column offsets per unit of z0, z1
  long long o1_n0, o1_n1;                // out1 column offsets per unit of z0, z1 (PoPE layout)
  long long o1_imag;                     // PoPE: column distance from the real to the imaginary half
  float alpha;
  float theta;
  int T;                 // sequence length: position of row m is pos0 + (m % T)
  int pos0;
  int n_per_head;        // rotary frequency index = column % n_per_head
  const float* freqs;    // [n_per_head] cycles per position
  const float* slopes;   // [nz0] decay slope per z0 (nullptr: no decay)
  int flags;
};

struct GemmArgs {
  int M, N, K;
  int nz0, nz1;
  OperandOffsets a, b;
  int causal_tiles;  // 0: all tiles; 1: only tiles that touch s < t (n0 <= m0+BM-1); 2: only tiles with s > t
  int causal_k;      // 1: contract only k < m0 + BM
  EpiParams epi;
  int* status;
};

// ------------------------------------------------------------------------------------------------
// Row-wise global memory helpers: each epilogue thread owns one output row and 32 columns.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void store_bf16_32(__nv_bfloat16* base, long long ld, long long r,
                                              long long c, const float (&v)[32], int valid) {
  __nv_bfloat16* p = base + r * ld + c;
  if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
    uint4* p4 = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u;
      u.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
      u.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
      u.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
      u.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      p4[i] = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) p[i] = __float2bfloat16_rn(v[i]);
  }
}

__device__ __forceinline__ void load_bf16_32(const __nv_bfloat16* base, long long ld, long long r,
                                             long long c, float (&v)[32], int valid) {
  const __nv_bfloat16* p = base + r * ld + c;
  if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u = __ldg(p4 + i);
      float2 f;
      f = unpack_bf16x2(u.x); v[8 * i + 0] = f.x; v[8 * i + 1] = f.y;
      f = unpack_bf16x2(u.y); v[8 * i + 2] = f.x; v[8 * i + 3] = f.y;
      f = unpack_bf16x2(u.z); v[8 * i + 4] = f.x; v[8 * i + 5] = f.y;
      f = unpack_bf16x2(u.w); v[8 * i + 6] = f.x; v[8 * i + 7] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = (i < valid) ? __bfloat162float(p[i]) : 0.f;
  }
}

__device__ __forceinline__ void store_f32_32(float* base, long long ld, long long r, long long c,
                                             const float (&v)[32], int valid, bool accum) {
  float* p = base + r * ld + c;
  if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
    float4* p4 = reinterpret_cast<float4*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 u = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      if (accum) {
        float4 o = p4[i];
        u.x += o.x; u.y += o.y; u.z += o.z; u.w += o.w;
      }
      p4[i] = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) p[i] = accum ? p[i] + v[i] : v[i];
  }
}

// Rotary phase of (position, column): 2*pi*frac(pos * freq), as the reference computes it
// (src/model/attention.rs:332-349).
__device__ __forceinline__ void rot_sincos(float pos, float freq, float& s, float& c) {
  float raw = pos * freq;
  float ph = (raw - floorf(raw)) * 6.283185307179586f;
  __sincosf(ph, &s, &c);
}

// ------------------------------------------------------------------------------------------------
// Epilogue: v holds columns [n, n+32) of row m (both relative to the batch's C block).
// ------------------------------------------------------------------------------------------------
template <int EPI>
__device__ __forceinline__ void epilogue_apply(const EpiParams& e, int z0, int z1, int m, int n,
                                               float (&v)[32], int M, int N) {
  if (m >= M || n >= N) return;
  const int valid = min(32, N - n);
  const long long r = e.c_m0 * z0 + e.c_m1 * z1 + m;
  const long long c = e.c_n0 * z0 + e.c_n1 * z1 + n;

  if constexpr (EPI == EPI_STORE) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= e.alpha;
    if (e.flags & EPI_F_OUT_F32) {
      store_f32_32(static_cast<float*>(e.out0), e.ld_out0, r, c, v, valid, e.flags & EPI_F_ACCUM);
    } else {
      if (e.flags & EPI_F_ACCUM) {
        float o[32];
        load_bf16_32(static_cast<const __nv_bfloat16*>(e.out0), e.ld_out0, r, c, o, valid);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += o[i];
      }
      store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
    }
  } else if constexpr (EPI == EPI_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i] - e.theta, 0.f);
    store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
    if (e.flags & (EPI_F_ROPE | EPI_F_POPE)) {
      const float pos = static_cast<float>(e.pos0 + (m % e.T));
      const int fcol = n % e.n_per_head;
      const long long c1 = e.o1_n0 * z0 + e.o1_n1 * z1 + n;
      if (e.flags & EPI_F_ROPE) {
        float q[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float a = v[i], b = v[i + 1];
          if (a != 0.f || b != 0.f) {
            float s, co;
            rot_sincos(pos, __ldg(e.freqs + fcol + i), s, co);
            q[i] = a * co - b * s;
            q[i + 1] = b * co + a * s;
          } else {
            q[i] = 0.f;
            q[i + 1] = 0.f;
          }
        }
        store_bf16_32(static_cast<__nv_bfloat16*>(e.out1), e.ld_out1, r, c1, q, valid);
      } else {
        float re[32], im[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s, co;
          rot_sincos(pos, __ldg(e.freqs + fcol + i), s, co);
          // softplus of a non-negative value: x + log1p(exp(-x))
          float mag = v[i] + log1pf(__expf(-v[i]));
          re[i] = mag * co;
          im[i] = mag * s;
        }
        store_bf16_32(static_cast<__nv_bfloat16*>(e.out1), e.ld_out1, r, c1, re, valid);
        store_bf16_32(static_cast<__nv_bfloat16*>(e.out1), e.ld_out1, r, c1 + e.o1_imag, im, valid);
      }
    }
  } else if constexpr (EPI == EPI_RELU_GATE) {
    float x[32];
    load_bf16_32(static_cast<const __nv_bfloat16*>(e.in0), e.ld_in0, r, c, x, valid);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i] - e.theta, 0.f);
    if (!(e.flags & EPI_F_NO_OUT0))
      store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= x[i];
    store_bf16_32(static_cast<__nv_bfloat16*>(e.out1), e.ld_out1, r, c, v, valid);
  } else if constexpr (EPI == EPI_CAUSAL) {
    const float slope = e.slopes ? __ldg(e.slopes + z0) : 0.f;
    const bool upper = e.flags & EPI_F_UPPER;
    if (!upper) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        int s = n + i;
        float w = (s < m) ? __expf(-slope * static_cast<float>(m - s)) : 0.f;
        v[i] *= w * e.alpha;
      }
      store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
    } else {
      if (n + 31 <= m) return;  // nothing above the diagonal in this chunk
      __nv_bfloat16* p = static_cast<__nv_bfloat16*>(e.out0) + r * e.ld_out0 + c;
      if (n > m && valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          v[i] *= e.alpha * __expf(-slope * static_cast<float>(n + i - m));
        store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          int s = n + i;
          if (i < valid && s > m)
            p[i] = __float2bfloat16_rn(v[i] * e.alpha * __expf(-slope * static_cast<float>(s - m)));
        }
      }
    }
  } else if constexpr (EPI == EPI_GATE_BWD) {
    float x[32], y[32];
    load_bf16_32(static_cast<const __nv_bfloat16*>(e.in0), e.ld_in0, r, c, x, valid);
    load_bf16_32(static_cast<const __nv_bfloat16*>(e.in1), e.ld_in1, r, c, y, valid);
    float dy[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      dy[i] = (y[i] > 0.f) ? v[i] * x[i] : 0.f;
      v[i] *= y[i];
    }
    store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, dy, valid);
    store_bf16_32(static_cast<__nv_bfloat16*>(e.out1), e.ld_out1, r, c, v, valid);
  } else if constexpr (EPI == EPI_DQ_BWD) {
    float x[32];
    load_bf16_32(static_cast<const __nv_bfloat16*>(e.in0), e.ld_in0, r, c, x, valid);
    if (e.flags & EPI_F_ROPE) {
      // q = R(pos) x  =>  dx = R(pos)^T dq
      const float pos = static_cast<float>(e.pos0 + (m % e.T));
      const int fcol = n % e.n_per_head;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        if (x[i] > 0.f || x[i + 1] > 0.f) {
          float s, co;
          rot_sincos(pos, __ldg(e.freqs + fcol + i), s, co);
          float a = v[i], b = v[i + 1];
          v[i] = a * co + b * s;
          v[i + 1] = b * co - a * s;
        }
      }
    }
    if (e.flags & EPI_F_HAS_IN1) {
      float g[32];
      load_bf16_32(static_cast<const __nv_bfloat16*>(e.in1), e.ld_in1, r, c, g, valid);
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += g[i];
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = (x[i] > 0.f) ? v[i] * e.alpha : 0.f;
    store_bf16_32(static_cast<__nv_bfloat16*>(e.out0), e.ld_out0, r, c, v, valid);
  }
}

// ------------------------------------------------------------------------------------------------
// Tile enumeration shared by the three roles (they must agree on the sequence).
// ------------------------------------------------------------------------------------------------
struct TileCoord {
  int z0, z1, m0, n0;
};

template <int BN>
struct TileWalker {
  int tiles_m, tiles_n, per_z, total, nz0, mode;
  __device__ TileWalker(const GemmArgs& g) {
    tiles_m = (g.M + GEMM_BM - 1) / GEMM_BM;
    tiles_n = (g.N + BN - 1) / BN;
    nz0 = g.nz0;
    mode = g.causal_tiles;
    if (mode == 0) {
      per_z = tiles_m * tiles_n;
    } else {
      per_z = 0;
      for (int mi = 0; mi < tiles_m; ++mi) per_z += count(mi);
    }
    total = per_z * g.nz0 * g.nz1;
  }
  __device__ __forceinline__ int first(int mi) const {
    return (mode == 2) ? min(tiles_n, (mi * GEMM_BM) / BN) : 0;
  }
  __device__ __forceinline__ int count(int mi) const {
    if (mode == 1) return min(tiles_n, (mi * GEMM_BM + GEMM_BM - 1) / BN + 1);
    if (mode == 2) return tiles_n - first(mi);
    return tiles_n;
  }
  __device__ __forceinline__ TileCoord decode(int t) const {
    TileCoord tc;
    int z = t / per_z, r = t - z * per_z;
    tc.z0 = z % nz0;
    tc.z1 = z / nz0;
    int mi, ni;
    if (mode == 0) {
      mi = r / tiles_n;
      ni = r - mi * tiles_n;
    } else {
      mi = 0;
      while (r >= count(mi)) {
        r -= count(mi);
        ++mi;
      }
      ni = first(mi) + r;
    }
    tc.m0 = mi * GEMM_BM;
    tc.n0 = ni * BN;
    return tc;
  }
};

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 5) * 8 + 16 + 1024;  // +1024: manual alignment slack
};

template <int BN, int A_MN, int B_MN, int EPI, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmArgs g) {
  using L = GemmSmem<BN, STAGES>;
  static_assert(BN == 128 || BN == 256, "BN must be 128 or 256");
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* drain_bar = tempty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], GEMM_EPI_WARPS);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const TileWalker<BN> walker(g);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t armed = 0, armed_parity = 0;  // per-stage: a load was issued / with which phase
      for (int t = blockIdx.x; t < walker.total && ok; t += gridDim.x) {
        const TileCoord tc = walker.decode(t);
        const int k_end = g.causal_k ? min(g.K, tc.m0 + GEMM_BM) : g.K;
        const int nkb = (k_end + GEMM_BK - 1) / GEMM_BK;
        const int a_mn = static_cast<int>(tc.m0 + tc.z0 * g.a.mn0 + tc.z1 * g.a.mn1);
        const int a_k = static_cast<int>(tc.z0 * g.a.k0 + tc.z1 * g.a.k1);
        const int b_mn = static_cast<int>(tc.n0 + tc.z0 * g.b.mn0 + tc.z1 * g.b.mn1);
        const int b_k = static_cast<int>(tc.z0 * g.b.k0 + tc.z1 * g.b.k1);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, g.status,
                         STATUS_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          const int kc = kb * GEMM_BK;
          if constexpr (A_MN == 0) {
            tma_load_2d(sa, &tmA, &full_bar[stage], a_k + kc, a_mn);
          } else {
#pragma unroll
            for (int i = 0; i < GEMM_BM / 64; ++i)
              tma_load_2d(sa + i * (GEMM_BK * 128), &tmA, &full_bar[stage], a_mn + i * 64, a_k + kc);
          }
          if constexpr (B_MN == 0) {
            tma_load_2d(sb, &tmB, &full_bar[stage], b_k + kc, b_mn);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sb + i * (GEMM_BK * 128), &tmB, &full_bar[stage], b_mn + i * 64, b_k + kc);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (*abort_flag) {
        // Gave up somewhere: let this thread's copies land before the CTA's memory goes away.
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&full_bar[s], (armed_parity >> s) & 1u)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < walker.total && ok; t += gridDim.x) {
        const TileCoord tc = walker.decode(t);
        const int k_end = g.causal_k ? min(g.K, tc.m0 + GEMM_BM) : g.K;
        const int nkb = (k_end + GEMM_BK - 1) / GEMM_BK;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, g.status,
                       STATUS_TIMEOUT_TMEM_EMPTY))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t da = (A_MN == 0) ? make_smem_desc(sa + k * 32, 16, 1024)
                                            : make_smem_desc(sa + k * 2048, GEMM_BK * 128, 1024);
            const uint64_t db = (B_MN == 0) ? make_smem_desc(sb + k * 32, 16, 1024)
                                            : make_smem_desc(sb + k * 2048, GEMM_BK * 128, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (*abort_flag) {
        // Let the MMAs already issued retire before TMEM is released.
        umma_commit(drain_bar);
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(drain_bar, 0)) break;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < walker.total; t += gridDim.x) {
      const TileCoord tc = walker.decode(t);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL))
        break;
      tc_fence_after();
      const int m = tc.m0 + q * 32 + lane;
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        float v[32];
        tmem_ld_32x32(tbase + c * 32, v);
        tmem_ld_wait();
        epilogue_apply<EPI>(g.epi, tc.z0, tc.z1, m, tc.n0 + c * 32, v, g.M, g.N);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------- teardown (every path reaches this) ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace bdh
