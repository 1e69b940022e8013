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
// Epilogue warps: 4 (one per TMEM lane quarter) or 8 (two per quarter, each taking half of the
// tile's columns) - the second keeps two warps per scheduler busy when the epilogue is heavy.
constexpr int gemm_threads(int epi_warps) { return 32 * (2 + epi_warps); }

enum EpiKind : int {
  EPI_STORE = 0,       // out0 = alpha*acc (+ beta*out0); bf16 or fp32 by flag
  EPI_RELU = 1,        // x = relu(acc - theta) -> out0 ; optional q = rot(x) -> out1
  EPI_RELU_GATE = 2,   // y = relu(acc - theta) -> out0 (optional) ; xy = y * in0 -> out1
  EPI_CAUSAL = 3,      // out0 = mask(t, s) * acc * exp(-slope*|t-s|)
  EPI_GATE_BWD = 4,    // g = acc ; in0 = x, in1 = x*y ; out0 = g*x*[y>0] ; out1 = g*y*[x>0] (-0.0 marks closed)
  EPI_DQ_BWD = 5,      // dq = rot^-1(acc) ; in0 = marked gate gradient ; out0 = open ? dq + in0 : 0
};

enum EpiFlags : int {
  EPI_F_OUT_F32 = 1,       // EPI_STORE: out0 is fp32 (else bf16)
  EPI_F_ACCUM = 2,         // EPI_STORE: out0 += (beta = 1)
  EPI_F_ROPE = 4,          // EPI_RELU: also write the RoPE-rotated copy to out1; EPI_DQ_BWD: undo it
  EPI_F_POPE = 8,          // EPI_RELU: write softplus(x)*[cos, sin] to out1 (real | imag halves)
  EPI_F_UPPER = 16,        // EPI_CAUSAL: write only s > t (else: write everything, zero where s >= t)
  EPI_F_NO_OUT0 = 32,      // EPI_RELU_GATE: skip storing y
  EPI_F_BIAS = 64,         // EPI_CAUSAL: additive distance bias, acc + slope*(s-t), instead of the decay factor
  EPI_F_TABLE = 128,       // rotary (cos, sin) come from an fp16-pair table [T, n_per_head] instead of sincos
  EPI_F_ATOMIC = 512,      // EPI_STORE fp32: out0 += tile with red.global.add (split-K partial sums)
  EPI_F_MC_RED = 256,      // EPI_STORE fp32: out0 is an NVSwitch multicast address; add the tile into every
                           // rank's replica with multimem.red (tensor-parallel partial-sum reduction)
  EPI_F_ROWDECAY = 2048,   // EPI_STORE: scale row m by exp(-slopes[z0] * m) (decayed carry-in of a recurrent state)
  EPI_F_ROWDECAY_REV = 8192,  // EPI_STORE: scale row m by exp(-slopes[z0] * (T - m)): what a row still contributes
                              // to the state at the end of a segment of T rows (gradient of the segment state)
  EPI_F_KEEP_MARK = 4096,  // EPI_DQ_BWD: closed gates keep their -0.0 marker in out0 (instead of 0), so that a
                           // second EPI_DQ_BWD launch can take out0 as its in0 and add another product
  EPI_F_PEER_RS = 1024,    // EPI_STORE fp32: reduce-scatter epilogue (with EPI_F_ATOMIC: add into the owner's
                           // single block instead of storing into a per-rank slot). Output rows are split into blocks of
                           // peer_rows, block b is owned by rank b. The tile is stored through the owner's
                           // peer mapping peer_out[owner] into the slot this rank has there: the owner's
                           // buffer is [world slots][peer_rows][ld] and slot s receives rank s's partial
                           // sums, which the owner adds up afterwards (collectives.cu: gather_blocks)
};

constexpr int GEMM_MAX_PEERS = 8;

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
  const float* bias;     // EPI_RELU / EPI_RELU_GATE: fp32 bias per output column (C coordinates), added before
                         // the threshold (reference: src/kernel/relu_lowrank.rs:19-23); nullptr: none
  int flags;
  float drop_p;          // EPI_RELU_GATE: dropout probability applied to x*y (0: off)
  uint32_t drop_seed;    // EPI_RELU_GATE: seed of the counter-based dropout mask
  float* peer_out[GEMM_MAX_PEERS];   // EPI_F_PEER_RS: every rank's mapping of the (symmetric) slot buffer
  long long peer_rows;               // EPI_F_PEER_RS: rows per owner block
  int peer_world, peer_rank;
};

// All-gather of the A operand inside the GEMM (token-sharded activations under tensor parallelism): every rank
// holds the rows [r * shard_rows, (r + 1) * shard_rows) of A in its own copy of a symmetric [M, K] buffer. At the
// start of the kernel the epilogue warps of all CTAs pull the other ranks' row blocks (128 rows each) over NVLink
// into the local copy with plain peer loads, in ring order from the next rank on, and count every finished block
// in `arrived`; the TMA producer loads a row block of A (from LOCAL memory) only once its counter has reached
// `target`. Tiles are walked from the local rows on (tile_shift), so the math on the rows that are already here
// overlaps the transfer of the others. world <= 1: no gather.
struct GatherArgs {
  const uint4* src[GEMM_MAX_PEERS];   // every rank's copy of the buffer (peer mappings; [rank] is unused)
  uint4* dst;                         // this rank's copy (the A tensor map points at it)
  long long block_vec;                // 16-byte vectors per block of GEMM_BM rows
  int blocks_per_shard;
  unsigned* arrived;                  // [M / GEMM_BM] counters, zero before the launch
  unsigned target;                    // counter value of a complete block (= number of epilogue warps)
  int world, rank;
};

struct GemmArgs {
  GatherArgs gather;
  int M, N, K;
  int nz0, nz1;
  OperandOffsets a, b;
  int causal_tiles;  // 0: all tiles; 1: only tiles that touch s < t (n0 <= m0+BM-1); 2: only tiles with s > t
  int causal_k;      // 1: contract only k < m0 + BM; 2: only k >= m0 (m0 = first row of the tile); the K
                     // range is never empty as long as K > the last tile's first row
  const unsigned char* tile_skip;   // EPI_CAUSAL: [tiles_m, tiles_n] bytes, non-zero = this output tile is not computed
                                    // and not written (an inactive pair of time blocks); nullptr: every tile runs
  int l2_hints;      // 1: the staged epilogue's output stores and streamed aux loads carry L2 evict_first, the
                     // operand loads of the small-operand epilogues (EPI 1, 2, 4) evict_last: the [tokens, neurons]
                     // streams then pass through L2 without pushing the weights out
  int tile_shift;    // tiles are visited in the order (t + tile_shift) mod total (reduce-scatter epilogue:
                     // each rank starts at another owner's rows so that no GPU is everybody's target)
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

// RoPE frequencies arrive as a pair table (one entry per (2i, 2i+1) column pair, n_per_head/2
// entries); a 32-column chunk starting at column `col` uses 16 consecutive entries.
__device__ __forceinline__ void load_pair_freqs(const float* freqs, int col, float (&fr)[16]) {
  const float4* p = reinterpret_cast<const float4*>(freqs + (col >> 1));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 f = __ldg(p + i);
    fr[4 * i] = f.x; fr[4 * i + 1] = f.y; fr[4 * i + 2] = f.z; fr[4 * i + 3] = f.w;
  }
}

// ------------------------------------------------------------------------------------------------
// Epilogue math on registers. `acc` holds columns [n, n+32) of row m (both relative to the batch's
// C block); r0 / r1 are the matching 32 auxiliary values as packed bf16 pairs (or fp16 cos/sin
// pairs for the rotary table); results go to o0 / o1. Which of the four are live for an
// (EPI, flags) pair is given by epi_io_mask().
//
// Gradient encoding shared by EPI_GATE_BWD and EPI_DQ_BWD: the gate gradient w.r.t. x is stored
// with the bf16 bit pattern of -0.0 wherever the ReLU that produced x is closed (x <= 0). The
// consumer masks by that marker instead of re-reading x.
// ------------------------------------------------------------------------------------------------
enum : int { IO_IN0 = 1, IO_IN1 = 2, IO_OUT0 = 4, IO_OUT1 = 8, IO_OUT2 = 16 };   // OUT2: PoPE imaginary half (in out1)
constexpr uint32_t BF16_NEG_ZERO = 0x8000u;

__host__ __device__ inline int epi_io_mask(int epi, int flags) {
  switch (epi) {
    case EPI_STORE: return IO_OUT0;
    case EPI_RELU:
      return IO_OUT0 | ((flags & (EPI_F_ROPE | EPI_F_POPE)) ? IO_OUT1 : 0) | ((flags & EPI_F_POPE) ? IO_OUT2 : 0) |
             (((flags & EPI_F_ROPE) && (flags & EPI_F_TABLE)) ? IO_IN0 : 0);
    case EPI_RELU_GATE: return IO_IN0 | IO_OUT1 | ((flags & EPI_F_NO_OUT0) ? 0 : IO_OUT0);
    case EPI_CAUSAL: return IO_OUT0;
    case EPI_GATE_BWD: return IO_IN0 | IO_IN1 | IO_OUT0 | IO_OUT1;
    case EPI_DQ_BWD:
      return IO_IN0 | IO_OUT0 | (((flags & EPI_F_ROPE) && (flags & EPI_F_TABLE)) ? IO_IN1 : 0);
  }
  return 0;
}

// Epilogues whose outputs are plain bf16 tiles at C's coordinates can be staged through shared
// memory and moved with TMA; the others (fp32 / accumulate / PoPE layout / partial upper writes)
// use per-thread global accesses.
__host__ __device__ inline bool epi_tma_capable(int epi, int flags) {
  if (epi == EPI_STORE)
    return !(flags & (EPI_F_OUT_F32 | EPI_F_ACCUM | EPI_F_MC_RED | EPI_F_ATOMIC | EPI_F_PEER_RS | EPI_F_ROWDECAY |
                      EPI_F_ROWDECAY_REV));
  if (epi == EPI_RELU) return true;
  if (epi == EPI_CAUSAL) return !(flags & EPI_F_UPPER);
  return true;
}

__device__ __forceinline__ float2 unpack_f16x2(uint32_t u) {
  __half2 h = *reinterpret_cast<__half2*>(&u);
  return __half22float2(h);
}

// (cos, sin) of the rotary phase for the 16 column pairs of a chunk: from the table (fp16 pairs in
// `tab`) or computed from the pair-frequency list.
template <bool TABLE>
__device__ __forceinline__ void rot_pair(const EpiParams& e, const uint32_t (&tab)[16], const float (&fr)[16],
                                         float pos, int i, float& s, float& co) {
  if (TABLE) {
    float2 cs = unpack_f16x2(tab[i]);
    co = cs.x;
    s = cs.y;
  } else {
    rot_sincos(pos, fr[i], s, co);
  }
}

__device__ __forceinline__ uint32_t dropout_hash(uint32_t h) {
  h ^= h >> 16; h *= 0x7feb352du; h ^= h >> 15; h *= 0x846ca68bu; h ^= h >> 16;
  return h;
}

template <int EPI>
__device__ __forceinline__ void epi_compute(const EpiParams& e, int z0, int m, int n, float (&acc)[32],
                                            const uint32_t (&r0)[16], const uint32_t (&r1)[16],
                                            float (&o0)[32], float (&o1)[32], float (&o2)[32]) {
  if constexpr (EPI == EPI_STORE) {
#pragma unroll
    for (int i = 0; i < 32; ++i) o0[i] = acc[i] * e.alpha;
  } else if constexpr (EPI == EPI_RELU) {
#pragma unroll
    for (int i = 0; i < 32; ++i) o0[i] = fmaxf(acc[i] - e.theta, 0.f);
    if (e.flags & EPI_F_POPE) {
      // q = softplus(x) * (cos, sin): real half -> o1, imaginary half -> o2
      const float pos = static_cast<float>(e.pos0 + (m % e.T));
      const float4* fp = reinterpret_cast<const float4*>(e.freqs + (n % e.n_per_head));
#pragma unroll
      for (int i4 = 0; i4 < 8; ++i4) {
        const float4 f = __ldg(fp + i4);
        const float fr[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = 4 * i4 + j;
          float s, co;
          rot_sincos(pos, fr[j], s, co);
          const float mag = o0[i] + __logf(1.f + __expf(-o0[i]));   // softplus of a non-negative value
          o1[i] = mag * co;
          o2[i] = mag * s;
        }
      }
    } else if (e.flags & EPI_F_ROPE) {
      if (e.flags & EPI_F_TABLE) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 cs = unpack_f16x2(r0[i]);
          float a = o0[2 * i], b = o0[2 * i + 1];
          o1[2 * i] = a * cs.x - b * cs.y;
          o1[2 * i + 1] = b * cs.x + a * cs.y;
        }
      } else {
        const float pos = static_cast<float>(e.pos0 + (m % e.T));
        float fr[16];
        load_pair_freqs(e.freqs, n % e.n_per_head, fr);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float a = o0[2 * i], b = o0[2 * i + 1];
          if (a != 0.f || b != 0.f) {
            float s, co;
            rot_sincos(pos, fr[i], s, co);
            o1[2 * i] = a * co - b * s;
            o1[2 * i + 1] = b * co + a * s;
          } else {
            o1[2 * i] = 0.f;
            o1[2 * i + 1] = 0.f;
          }
        }
      }
    }
  } else if constexpr (EPI == EPI_RELU_GATE) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 x = unpack_bf16x2(r0[i]);
      o0[2 * i] = fmaxf(acc[2 * i] - e.theta, 0.f);
      o0[2 * i + 1] = fmaxf(acc[2 * i + 1] - e.theta, 0.f);
      o1[2 * i] = o0[2 * i] * x.x;
      o1[2 * i + 1] = o0[2 * i + 1] * x.y;
    }
    if (e.drop_p > 0.f) {
      // inverted dropout on x*y (reference: src/model/bdh.rs:380-381). One 32-bit hash of
      // (seed, z0, row, column pair) gives two 16-bit uniforms; kept values are scaled by 1/(1-p).
      const uint32_t thr = static_cast<uint32_t>(e.drop_p * 65536.f);
      const float keep_scale = 1.f / (1.f - e.drop_p);
      const uint32_t base = e.drop_seed ^ (static_cast<uint32_t>(m) * 0x9E3779B1u) ^
                            (static_cast<uint32_t>(z0) * 0xC2B2AE3Du);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t h = dropout_hash(base ^ (static_cast<uint32_t>((n >> 1) + i) * 0x85EBCA77u));
        o1[2 * i] = ((h & 0xFFFFu) >= thr) ? o1[2 * i] * keep_scale : 0.f;
        o1[2 * i + 1] = ((h >> 16) >= thr) ? o1[2 * i + 1] * keep_scale : 0.f;
      }
    }
  } else if constexpr (EPI == EPI_CAUSAL) {
    const float slope = e.slopes ? __ldg(e.slopes + z0) : 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      int s = n + i;
      if (e.flags & EPI_F_BIAS) {
        o0[i] = (s < m) ? acc[i] * e.alpha - slope * static_cast<float>(m - s) : 0.f;
      } else {
        float w = (s < m) ? __expf(-slope * static_cast<float>(m - s)) : 0.f;
        o0[i] = acc[i] * w * e.alpha;
      }
    }
  } else if constexpr (EPI == EPI_GATE_BWD) {
    // r0 = x, r1 = x*y (y itself is never stored: y = xy / x where the x gate is open).
    //   o0 = d(pre-activation of y) = g * x where y > 0   (y > 0  <=>  xy > 0 because x >= 0)
    //   o1 = gate gradient w.r.t. x = g * y where x > 0, else the -0.0 marker
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 x = unpack_bf16x2(r0[i]);
      float2 xy = unpack_bf16x2(r1[i]);
      o0[2 * i] = (xy.x > 0.f) ? acc[2 * i] * x.x * e.alpha : 0.f;
      o0[2 * i + 1] = (xy.y > 0.f) ? acc[2 * i + 1] * x.y * e.alpha : 0.f;
      float g0 = acc[2 * i] * __fdividef(xy.x, x.x), g1 = acc[2 * i + 1] * __fdividef(xy.y, x.y);
      // +0.0 keeps "open gate, zero gradient" distinct from the marker
      o1[2 * i] = (x.x > 0.f) ? (g0 == 0.f ? 0.f : g0) : -0.f;
      o1[2 * i + 1] = (x.y > 0.f) ? (g1 == 0.f ? 0.f : g1) : -0.f;
    }
  } else if constexpr (EPI == EPI_DQ_BWD) {
    // r0 = gate gradient with -0.0 markers; r1 = rotary table (optional)
    if (e.flags & EPI_F_ROPE) {
      // q = R(pos) x  =>  dx = R(pos)^T dq
      const bool table = e.flags & EPI_F_TABLE;
      if (table) {
        // branch-free: four FMAs per pair are cheaper than a divergent skip
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 cs = unpack_f16x2(r1[i]);
          const float a = acc[2 * i], b = acc[2 * i + 1];
          acc[2 * i] = a * cs.x + b * cs.y;
          acc[2 * i + 1] = b * cs.x - a * cs.y;
        }
      } else {
        const float pos = static_cast<float>(e.pos0 + (m % e.T));
        float fr[16];
        load_pair_freqs(e.freqs, n % e.n_per_head, fr);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool closed = ((r0[i] & 0xFFFFu) == BF16_NEG_ZERO) && ((r0[i] >> 16) == BF16_NEG_ZERO);
          if (!closed) {
            float s, co;
            rot_sincos(pos, fr[i], s, co);
            float a = acc[2 * i], b = acc[2 * i + 1];
            acc[2 * i] = a * co + b * s;
            acc[2 * i + 1] = b * co - a * s;
          }
        }
      }
    }
    const float closed_val = (e.flags & EPI_F_KEEP_MARK) ? -0.f : 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float2 g = unpack_bf16x2(r0[i]);
      // (+ 0.f turns a computed -0.0 into +0.0: only closed gates may carry the marker)
      o0[2 * i] = ((r0[i] & 0xFFFFu) == BF16_NEG_ZERO) ? closed_val : acc[2 * i] * e.alpha + g.x + 0.f;
      o0[2 * i + 1] = ((r0[i] >> 16) == BF16_NEG_ZERO) ? closed_val : acc[2 * i + 1] * e.alpha + g.y + 0.f;
    }
  }
}

__device__ __forceinline__ void load_raw_32(const __nv_bfloat16* base, long long ld, long long r, long long c,
                                            uint32_t (&u)[16], int valid) {
  const __nv_bfloat16* p = base + r * ld + c;
  if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 w = __ldg(p4 + i);
      u[4 * i] = w.x; u[4 * i + 1] = w.y; u[4 * i + 2] = w.z; u[4 * i + 3] = w.w;
    }
  } else {
    const unsigned short* ps = reinterpret_cast<const unsigned short*>(p);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint32_t lo = (2 * i < valid) ? ps[2 * i] : 0u, hi = (2 * i + 1 < valid) ? ps[2 * i + 1] : 0u;
      u[i] = lo | (hi << 16);
    }
  }
}

constexpr int EPI_RED_FLAGS = EPI_F_MC_RED | EPI_F_ATOMIC | EPI_F_PEER_RS;

// Scale applied by EPI_STORE to row m of problem (z0, .): alpha, times the row decay when asked for.
__device__ __forceinline__ float epi_store_scale(const EpiParams& e, int z0, int m) {
  float a = e.alpha;
  if (e.flags & EPI_F_ROWDECAY) a *= __expf(-(e.slopes ? __ldg(e.slopes + z0) : 0.f) * static_cast<float>(m));
  if (e.flags & EPI_F_ROWDECAY_REV)
    a *= __expf(-(e.slopes ? __ldg(e.slopes + z0) : 0.f) * static_cast<float>(e.T - m));
  return a;
}

// Address of output row `row` inside the slot this rank owns in the buffer of the row's owner.
// With EPI_F_ATOMIC the owner keeps ONE block of peer_rows rows that every rank adds into (red.add over
// NVLink): the sharded gradient accumulator of fully sharded data parallelism, where each weight-gradient
// GEMM of each layer adds its tiles straight into the 1/world slice its owner holds.
__device__ __forceinline__ float* peer_slot_row(const EpiParams& e, long long row) {
  long long owner = row / e.peer_rows;
  if (owner >= e.peer_world) owner = e.peer_world - 1;
  const long long slot = (e.flags & EPI_F_ATOMIC) ? 0 : e.peer_rank * e.peer_rows;
  return e.peer_out[owner] + (slot + (row - owner * e.peer_rows)) * e.ld_out0;
}

__device__ __forceinline__ void red_add_f32x4(float* p, const float4& u, int flags) {
  if (flags & EPI_F_MC_RED)
    asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(u.x), "f"(u.y),
                 "f"(u.z), "f"(u.w)
                 : "memory");
  else
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(u.x), "f"(u.y), "f"(u.z), "f"(u.w)
                 : "memory");
}

// Sends one warp's full 32x32 fp32 tile (thread = row, v = its 32 columns) to global, multicast or
// peer memory: a reduction-add (EPI_F_ATOMIC, EPI_F_MC_RED) or a plain store into the owner's slot
// (EPI_F_PEER_RS). The tile is transposed through 4 KB of shared memory (16-byte slots, XOR-swizzled
// by row) so that 8 lanes cover one 128-byte row segment: every request that leaves the SM - and,
// for peer and multicast targets, every NVLink packet - carries a full 128 bytes instead of 16.
// r0 = output row of lane 0, c = first output column; the caller has checked 16-byte alignment.
// `add_local` (EPI_F_PEER_RS | EPI_F_ATOMIC | EPI_F_ACCUM, first K split only): the tile first takes up what the
// local fp32 buffer out0 holds at its position - the sum over the shared-weight layers processed before -
// so that one send per step carries the whole local gradient to its owner.
__device__ __forceinline__ void send_tile_coalesced(const EpiParams& e, long long r0, long long c,
                                                    const float (&v)[32], float4* scratch, int lane,
                                                    bool add_local = false) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
    scratch[lane * 8 + (i ^ (lane & 7))] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  __syncwarp();
  const int sub = lane >> 3, ch = lane & 7;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int row = 4 * j + sub;
    float4 u = scratch[row * 8 + (ch ^ (row & 7))];
    const long long rr = r0 + row;
    if (add_local) {
      const float4 l = *reinterpret_cast<const float4*>(static_cast<const float*>(e.out0) + rr * e.ld_out0 + c + 4 * ch);
      u.x += l.x; u.y += l.y; u.z += l.z; u.w += l.w;
    }
    if ((e.flags & EPI_F_PEER_RS) && (e.flags & EPI_F_ATOMIC))
      red_add_f32x4(peer_slot_row(e, rr) + c + 4 * ch, u, e.flags);
    else if (e.flags & EPI_F_PEER_RS)
      *reinterpret_cast<float4*>(peer_slot_row(e, rr) + c + 4 * ch) = u;
    else
      red_add_f32x4(static_cast<float*>(e.out0) + rr * e.ld_out0 + c + 4 * ch, u, e.flags);
  }
  __syncwarp();
}

// Per-thread global-memory epilogue (any shape, any alignment, every flag).
template <int EPI>
__device__ __forceinline__ void epilogue_direct(const EpiParams& e, int z0, int z1, int m, int n,
                                                float (&v)[32], int M, int N) {
  if (m >= M || n >= N) return;
  const int valid = min(32, N - n);
  const long long r = e.c_m0 * z0 + e.c_m1 * z1 + m;
  const long long c = e.c_n0 * z0 + e.c_n1 * z1 + n;
  typedef __nv_bfloat16 bf;

  if constexpr (EPI == EPI_STORE) {
    const float scale = epi_store_scale(e, z0, m);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= scale;
    if (e.flags & EPI_F_MC_RED) {
      // partial sums of all ranks meet in the switch: one reduction-add per 16 bytes, no local read
      float* p = static_cast<float*>(e.out0) + r * e.ld_out0 + c;
      if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4 * i),
                       "f"(v[4 * i]), "f"(v[4 * i + 1]), "f"(v[4 * i + 2]), "f"(v[4 * i + 3])
                       : "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < valid)
            asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p + i), "f"(v[i]) : "memory");
      }
    } else if ((e.flags & EPI_F_PEER_RS) && (e.flags & EPI_F_ATOMIC)) {
      float* p = peer_slot_row(e, r) + c;
      const float* l = ((e.flags & EPI_F_ACCUM) && z1 == 0) ? static_cast<const float*>(e.out0) + r * e.ld_out0 + c : nullptr;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < valid) atomicAdd(p + i, l ? v[i] + l[i] : v[i]);
    } else if (e.flags & EPI_F_PEER_RS) {
      float* p = peer_slot_row(e, r) + c;
      if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < valid) p[i] = v[i];
      }
    } else if (e.flags & EPI_F_ATOMIC) {
      float* p = static_cast<float*>(e.out0) + r * e.ld_out0 + c;
      if (valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p + 4 * i), "f"(v[4 * i]),
                       "f"(v[4 * i + 1]), "f"(v[4 * i + 2]), "f"(v[4 * i + 3])
                       : "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < valid) atomicAdd(p + i, v[i]);
      }
    } else if (e.flags & EPI_F_OUT_F32) {
      store_f32_32(static_cast<float*>(e.out0), e.ld_out0, r, c, v, valid, e.flags & EPI_F_ACCUM);
    } else {
      if (e.flags & EPI_F_ACCUM) {
        float o[32];
        load_bf16_32(static_cast<const bf*>(e.out0), e.ld_out0, r, c, o, valid);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += o[i];
      }
      store_bf16_32(static_cast<bf*>(e.out0), e.ld_out0, r, c, v, valid);
    }
    return;
  }
  if constexpr (EPI == EPI_CAUSAL) {
    if (e.flags & EPI_F_UPPER) {
      if (n + 31 <= m) return;  // nothing above the diagonal in this chunk
      const float slope = e.slopes ? __ldg(e.slopes + z0) : 0.f;
      bf* p = static_cast<bf*>(e.out0) + r * e.ld_out0 + c;
      if (n > m && valid >= 32 && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
        // the whole chunk lies above the diagonal: vector stores
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= e.alpha * __expf(-slope * static_cast<float>(n + i - m));
        store_bf16_32(static_cast<bf*>(e.out0), e.ld_out0, r, c, v, valid);
        return;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        int s = n + i;
        if (i < valid && s > m)
          p[i] = __float2bfloat16_rn(v[i] * e.alpha * __expf(-slope * static_cast<float>(s - m)));
      }
      return;
    }
  }
  const int io = epi_io_mask(EPI, e.flags);
  uint32_t r0[16], r1[16];
  float o0[32], o1[32], o2[32];
  if constexpr (EPI == EPI_RELU || EPI == EPI_RELU_GATE) {
    if (e.bias) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < valid) v[i] += __ldg(e.bias + c + i);
    }
  }
  const bool tab0 = (EPI == EPI_RELU), tab1 = (EPI == EPI_DQ_BWD);   // which input is the rotary table
  // (the table row is the position of the OUTPUT row: batched problems that are segments of one sequence
  // - rows z1 * c_m1 + m - find their place in a table of the whole sequence)
  const long long tr = ((EPI == EPI_DQ_BWD) ? r : static_cast<long long>(m)) % e.T, tcn = n % e.n_per_head;
  if (io & IO_IN0)
    load_raw_32(static_cast<const bf*>(e.in0), e.ld_in0, tab0 ? tr : r, tab0 ? tcn : c, r0, valid);
  if (io & IO_IN1)
    load_raw_32(static_cast<const bf*>(e.in1), e.ld_in1, tab1 ? tr : r, tab1 ? tcn : c, r1, valid);
  epi_compute<EPI>(e, z0, m, n, v, r0, r1, o0, o1, o2);
  if (io & IO_OUT0) store_bf16_32(static_cast<bf*>(e.out0), e.ld_out0, r, c, o0, valid);
  if (io & IO_OUT1) {
    const long long c1 = (EPI == EPI_RELU) ? e.o1_n0 * z0 + e.o1_n1 * z1 + n : c;
    store_bf16_32(static_cast<bf*>(e.out1), e.ld_out1, r, c1, o1, valid);
    if (io & IO_OUT2) store_bf16_32(static_cast<bf*>(e.out1), e.ld_out1, r, c1 + e.o1_imag, o2, valid);
  }
}

// ---- shared-memory staging for the TMA epilogue ------------------------------------------------
// One [32 rows][32 bf16] box per (tensor, buffer): 64-byte rows with the 64-byte TMA swizzle
// (16-byte chunk index XOR bits 7-8 of the address). Thread `row` reads / writes its own row.
constexpr int EPI_BOX_BYTES = 32 * 64;
__device__ __forceinline__ uint32_t epi_box_off(int row, int chunk) {
  return static_cast<uint32_t>(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}
__device__ __forceinline__ void box_read_raw(const uint8_t* box, int row, uint32_t (&u)[16]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 w = *reinterpret_cast<const uint4*>(box + epi_box_off(row, j));
    u[4 * j] = w.x; u[4 * j + 1] = w.y; u[4 * j + 2] = w.z; u[4 * j + 3] = w.w;
  }
}
__device__ __forceinline__ void box_write_row(uint8_t* box, int row, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u;
    u.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
    u.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
    u.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
    u.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(box + epi_box_off(row, j)) = u;
  }
}

struct EpiMaps {
  CUtensorMap out0, out1, in0, in1;   // boxes of 32 columns x 32 rows, 64-byte swizzle
};

// ------------------------------------------------------------------------------------------------
// All-gather of A inside the kernel (GatherArgs).
// ------------------------------------------------------------------------------------------------
// Called by every epilogue warp of every CTA before its tile loop. Block u of the (world - 1) * blocks_per_shard
// remote blocks goes to CTA u % gridDim.x; the shards are taken in ring order from rank + 1 on, which is the
// order in which the tile walk reaches them.
__device__ __forceinline__ void gather_copy(const GatherArgs& ga, int ew, int n_warps, int lane) {
  const int units = (ga.world - 1) * ga.blocks_per_shard;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int s = u / ga.blocks_per_shard, j = u - s * ga.blocks_per_shard;
    int r = ga.rank + 1 + s;
    if (r >= ga.world) r -= ga.world;
    const long long blk = static_cast<long long>(r) * ga.blocks_per_shard + j;
    const uint4* src = ga.src[r] + blk * ga.block_vec;
    uint4* dst = ga.dst + blk * ga.block_vec;
    const long long step = static_cast<long long>(n_warps) * 32;
    long long i = static_cast<long long>(ew) * 32 + lane;
    // four loads in flight per thread: the peer round trip is a few microseconds
    for (; i + 3 * step < ga.block_vec; i += 4 * step) {
      const uint4 a = __ldcs(src + i), b = __ldcs(src + i + step), c = __ldcs(src + i + 2 * step),
                  d = __ldcs(src + i + 3 * step);
      dst[i] = a; dst[i + step] = b; dst[i + 2 * step] = c; dst[i + 3 * step] = d;
    }
    for (; i < ga.block_vec; i += step) dst[i] = __ldcs(src + i);
    __syncwarp();
    if (lane == 0) {
      __threadfence();                       // this warp's stores are visible before the count
      atomicAdd(ga.arrived + blk, 1u);
    }
  }
}

// Producer side: the block's counter has reached `target`, and the TMA unit (async proxy) may read what the
// copiers wrote with ordinary stores. Bounded like every other wait.
__device__ __forceinline__ bool gather_wait(const unsigned* counter, unsigned target, volatile int* abort_flag,
                                            int* status) {
  const uint64_t t0 = global_timer_ns();
  uint32_t it = 0;
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= target) break;
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > BDH_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicCAS(status, STATUS_OK, STATUS_TIMEOUT_PEER_FLAG);
        return false;
      }
    }
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// ------------------------------------------------------------------------------------------------
// Tile enumeration shared by the three roles (they must agree on the sequence).
// ------------------------------------------------------------------------------------------------
struct TileCoord {
  int z0, z1, m0, n0;
};

template <int BN>
struct TileWalker {
  int tiles_m, tiles_n, per_z, total, nz0, mode, shift;
  __device__ TileWalker(const GemmArgs& g) {
    shift = g.tile_shift;
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
    t += shift;
    if (t >= total) t -= total;
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

// Tile predicate of the causal epilogue (all three roles skip the same tiles, so the barrier phases stay in step).
template <int BN>
__device__ __forceinline__ bool tile_skipped(const GemmArgs& g, const TileCoord& tc) {
  if (!g.tile_skip) return false;
  const int tiles_n = (g.N + BN - 1) / BN;
  return g.tile_skip[(tc.m0 / GEMM_BM) * tiles_n + tc.n0 / BN] != 0;
}

// Boxes of staging per epilogue warp: double-buffered inputs and outputs.
__host__ __device__ constexpr int epi_num_in(int epi) {
  return (epi == EPI_RELU_GATE || epi == EPI_RELU) ? 1 : (epi == EPI_GATE_BWD || epi == EPI_DQ_BWD) ? 2 : 0;
}
__host__ __device__ constexpr int epi_num_out(int epi) {
  if (epi == EPI_RELU) return 3;       // x, rotated copy, PoPE imaginary half
  return (epi == EPI_RELU_GATE || epi == EPI_GATE_BWD) ? 2 : 1;
}

// Output boxes per tensor: the encoder epilogue (two or three outputs, bound by its HBM writes) keeps two, so
// a chunk can be written while the previous chunk's stores drain; the read-heavy epilogues keep one and give
// the shared memory to a third operand stage (the store of the previous chunk has long finished reading).
__host__ __device__ constexpr int epi_out_bufs(int epi) { return epi == EPI_RELU ? 2 : 1; }

constexpr int EPI_RED_TILE_BYTES = 32 * 32 * 4;

template <int BN, int STAGES, bool TMA_EPI, int EW, int EPI>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NIN = epi_num_in(EPI);
  static constexpr int NOUT = epi_num_out(EPI);
  // staged epilogue: 32x32 bf16 boxes per warp, two per auxiliary input (the next chunk's inputs are in
  // flight while this chunk is computed) and epi_out_bufs() per output; direct EPI_STORE: one 32x32 fp32 transposition tile per warp for the
  // coalesced reduction-add paths
  static constexpr int EPI_WARP_BYTES =
      TMA_EPI ? (2 * NIN + epi_out_bufs(EPI) * NOUT) * EPI_BOX_BYTES : (EPI == EPI_STORE ? EPI_RED_TILE_BYTES : 0);
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EW * EPI_WARP_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 5 + 2 * EW;
  static constexpr int TOTAL = BAR_OFFSET + NUM_BARS * 8 + 16 + 1024;  // +1024: manual alignment slack
};

template <int BN, int A_MN, int B_MN, int EPI, int STAGES, bool TMA_EPI, int EW>
__global__ void __launch_bounds__(gemm_threads(EW), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ EpiMaps em, const GemmArgs g) {
  using L = GemmSmem<BN, STAGES, TMA_EPI, EW, EPI>;
  static_assert(EW == 4 || EW == 8, "4 or 8 epilogue warps");
  constexpr int CHUNKS = (BN / 32) / (EW / 4);   // 32-column chunks per epilogue warp per tile
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
  uint64_t* in_bar = drain_bar + 1;  // [EW][2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(in_bar + 2 * EW);
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
      mbar_init(&tempty_bar[a], EW);
    }
    mbar_init(drain_bar, 1);
    for (int i = 0; i < 2 * EW; ++i) mbar_init(&in_bar[i], 1);
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
      int ready_block = -1;                  // last gathered row block known to be complete
      const uint64_t keep_policy = l2_policy_evict_last();
      for (int t = blockIdx.x; t < walker.total && ok; t += gridDim.x) {
        const TileCoord tc = walker.decode(t);
        if constexpr (EPI == EPI_CAUSAL) {
          if (tile_skipped<BN>(g, tc)) continue;
        }
        const int k_end = (g.causal_k == 1) ? min(g.K, tc.m0 + GEMM_BM) : g.K;
        const int nkb = (k_end + GEMM_BK - 1) / GEMM_BK;
        const int kb0 = (g.causal_k == 2) ? min(nkb, tc.m0 / GEMM_BK) : 0;
        if (g.gather.world > 1) {
          // rows of another rank: wait (bounded) until the copiers have brought the block into local memory
          const int blk = tc.m0 / GEMM_BM;
          if (blk / g.gather.blocks_per_shard != g.gather.rank && blk != ready_block) {
            if (!gather_wait(g.gather.arrived + blk, g.gather.target, abort_flag, g.status)) {
              ok = false;
              break;
            }
            ready_block = blk;
          }
        }
        const int a_mn = static_cast<int>(tc.m0 + tc.z0 * g.a.mn0 + tc.z1 * g.a.mn1);
        const int a_k = static_cast<int>(tc.z0 * g.a.k0 + tc.z1 * g.a.k1);
        const int b_mn = static_cast<int>(tc.n0 + tc.z0 * g.b.mn0 + tc.z1 * g.b.mn1);
        const int b_k = static_cast<int>(tc.z0 * g.b.k0 + tc.z1 * g.b.k1);
        for (int kb = kb0; kb < nkb; ++kb) {
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
          if constexpr (A_MN == 0 && B_MN == 0 && (EPI == EPI_RELU || EPI == EPI_RELU_GATE || EPI == EPI_GATE_BWD)) {
            if (g.l2_hints) {
              // both operands are small and re-read by every tile: keep them in L2
              tma_load_2d_hint(sa, &tmA, &full_bar[stage], a_k + kc, a_mn, keep_policy);
              tma_load_2d_hint(sb, &tmB, &full_bar[stage], b_k + kc, b_mn, keep_policy);
              if (++stage == STAGES) {
                stage = 0;
                phase ^= 1;
              }
              continue;
            }
          }
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
        if constexpr (EPI == EPI_CAUSAL) {
          if (tile_skipped<BN>(g, tc)) continue;
        }
        const int k_end = (g.causal_k == 1) ? min(g.K, tc.m0 + GEMM_BM) : g.K;
        const int nkb = (k_end + GEMM_BK - 1) / GEMM_BK;
        const int kb0 = (g.causal_k == 2) ? min(nkb, tc.m0 / GEMM_BK) : 0;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, g.status,
                       STATUS_TIMEOUT_TMEM_EMPTY))
          break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < nkb; ++kb) {
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
            umma_bf16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int ew = warp - 2;           // epilogue warp index
    const int cbase = (ew >> 2) * CHUNKS;   // first 32-column chunk of this warp inside a tile
    if (g.gather.world > 1) gather_copy(g.gather, ew, EW, lane);
    int acc = 0;
    uint32_t acc_phase = 0;
    if constexpr (!TMA_EPI) {
      for (int t = blockIdx.x; t < walker.total; t += gridDim.x) {
        const TileCoord tc = walker.decode(t);
        if constexpr (EPI == EPI_CAUSAL) {
          if (tile_skipped<BN>(g, tc)) continue;
        }
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL))
          break;
        tc_fence_after();
        const int m = tc.m0 + q * 32 + lane;
        const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
#pragma unroll 1
        for (int c = cbase; c < cbase + CHUNKS; ++c) {
          float v[32];
          tmem_ld_32x32(tbase + c * 32, v);
          tmem_ld_wait();
          if constexpr (EPI == EPI_STORE) {
            const EpiParams& e = g.epi;
            const int n = tc.n0 + c * 32;
            if ((e.flags & EPI_RED_FLAGS) && m - lane + 32 <= g.M && n + 32 <= g.N && (e.ld_out0 & 3) == 0) {
              const long long r0 = e.c_m0 * tc.z0 + e.c_m1 * tc.z1 + (m - lane);
              const long long cc = e.c_n0 * tc.z0 + e.c_n1 * tc.z1 + n;
              if (((reinterpret_cast<uintptr_t>(e.out0) + 4 * static_cast<uintptr_t>(cc)) & 15) == 0) {
                const float scale = epi_store_scale(e, tc.z0, m);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] *= scale;
                const bool add_local = (e.flags & EPI_F_PEER_RS) && (e.flags & EPI_F_ATOMIC) && (e.flags & EPI_F_ACCUM) &&
                                       tc.z1 == 0;
                send_tile_coalesced(e, r0, cc, v,
                                   reinterpret_cast<float4*>(smem + L::EPI_OFFSET + ew * L::EPI_WARP_BYTES), lane,
                                   add_local);
                continue;
              }
            }
          }
          epilogue_direct<EPI>(g.epi, tc.z0, tc.z1, m, tc.n0 + c * 32, v, g.M, g.N);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    } else {
      // Staged epilogue: auxiliary inputs arrive by TMA one 32-column chunk ahead, results leave by
      // TMA store; each warp owns its 32 rows end to end, so no cross-warp synchronisation is needed.
      const EpiParams& e = g.epi;
      const int io = epi_io_mask(EPI, e.flags);
      uint8_t* wbase = smem + L::EPI_OFFSET + ew * L::EPI_WARP_BYTES;
      uint8_t* in_box = wbase;                                   // [tensor][buf 0..1]
      uint8_t* out_box = wbase + 2 * L::NIN * EPI_BOX_BYTES;     // [tensor]
      uint64_t* ibar = in_bar + 2 * ew;
      const uint32_t in_bytes = ((io & IO_IN0) ? EPI_BOX_BYTES : 0) + ((io & IO_IN1) ? EPI_BOX_BYTES : 0);
      const bool has_in = in_bytes != 0;
      const uint64_t stream_policy = l2_policy_evict_first();
      uint32_t gchunk = 0;   // running chunk counter of this warp: buffer = gchunk & 1, parity = (gchunk >> 1) & 1
      uint32_t issued = 0;   // chunks whose input loads were issued

      auto issue_in = [&](const TileCoord& tc, int c) {
        // called by lane 0 only
        const int buf = issued & 1;
        const int row = static_cast<int>(e.c_m0 * tc.z0 + e.c_m1 * tc.z1 + tc.m0 + q * 32);
        const int col = static_cast<int>(e.c_n0 * tc.z0 + e.c_n1 * tc.z1 + tc.n0 + (cbase + c) * 32);
        // the rotary table is indexed by (position, column within the head), not by C coordinates
        const int trow = ((EPI == EPI_DQ_BWD) ? row : (tc.m0 + q * 32)) % e.T;
        const int tcol = (tc.n0 + (cbase + c) * 32) % e.n_per_head;
        mbar_arrive_expect_tx(&ibar[buf], in_bytes);
        // (the rotary table - in0 of EPI_RELU, in1 of EPI_DQ_BWD - is re-read by every tile; the other aux
        // inputs are [tokens, neurons] streams)
        if (io & IO_IN0) {
          if (g.l2_hints && EPI != EPI_RELU)
            tma_load_2d_hint(in_box + (0 * 2 + buf) * EPI_BOX_BYTES, &em.in0, &ibar[buf], col, row, stream_policy);
          else
            tma_load_2d(in_box + (0 * 2 + buf) * EPI_BOX_BYTES, &em.in0, &ibar[buf],
                        (EPI == EPI_RELU) ? tcol : col, (EPI == EPI_RELU) ? trow : row);
        }
        if (io & IO_IN1) {
          if (g.l2_hints && EPI != EPI_DQ_BWD)
            tma_load_2d_hint(in_box + (1 * 2 + buf) * EPI_BOX_BYTES, &em.in1, &ibar[buf], col, row, stream_policy);
          else
            tma_load_2d(in_box + (1 * 2 + buf) * EPI_BOX_BYTES, &em.in1, &ibar[buf],
                        (EPI == EPI_DQ_BWD) ? tcol : col, (EPI == EPI_DQ_BWD) ? trow : row);
        }
      };

      int t = blockIdx.x;
      TileCoord tc{0, 0, 0, 0};
      if (t < walker.total) {
        tc = walker.decode(t);
        if (has_in && lane == 0) issue_in(tc, 0);
        if (has_in) ++issued;
      }
      bool ok = true;
      while (t < walker.total && ok) {
        const int t_next = t + gridDim.x;
        TileCoord tc_next{0, 0, 0, 0};
        if (t_next < walker.total) tc_next = walker.decode(t_next);
        if constexpr (EPI == EPI_CAUSAL) {
          // (this epilogue has no auxiliary inputs, so nothing was prefetched for a skipped tile)
          if (tile_skipped<BN>(g, tc)) {
            t = t_next;
            tc = tc_next;
            continue;
          }
        }
        if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL))
          break;
        tc_fence_after();
        const int m = tc.m0 + q * 32 + lane;
        const uint32_t tbase = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
        const int row0 = static_cast<int>(e.c_m0 * tc.z0 + e.c_m1 * tc.z1 + tc.m0 + q * 32);
        const int col0 = static_cast<int>(e.c_n0 * tc.z0 + e.c_n1 * tc.z1 + tc.n0) + cbase * 32;
        const int col1 = (EPI == EPI_RELU) ? static_cast<int>(e.o1_n0 * tc.z0 + e.o1_n1 * tc.z1 + tc.n0) + cbase * 32 : col0;
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c, ++gchunk) {
          const int buf = gchunk & 1;
          float v[32], o0[32], o1[32], o2[32];
          uint32_t a0[16], a1[16];
          tmem_ld_32x32(tbase + (cbase + c) * 32, v);
          if (has_in) {
            if (!mbar_wait(&ibar[buf], (gchunk >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) {
              ok = false;
              tmem_ld_wait();
              break;
            }
            if (io & IO_IN0) box_read_raw(in_box + (0 * 2 + buf) * EPI_BOX_BYTES, lane, a0);
            if (io & IO_IN1) box_read_raw(in_box + (1 * 2 + buf) * EPI_BOX_BYTES, lane, a1);
            __syncwarp();
            // prefetch the next chunk (possibly the next tile's first) into the other buffer
            const bool more = (c + 1 < CHUNKS) || (t_next < walker.total);
            if (more) {
              if (lane == 0) {
                if (c + 1 < CHUNKS) issue_in(tc, c + 1);
                else issue_in(tc_next, 0);
              }
              ++issued;
            }
          }
          tmem_ld_wait();
          if constexpr (EPI == EPI_RELU || EPI == EPI_RELU_GATE) {
            if (e.bias) {
              const float4* bp = reinterpret_cast<const float4*>(e.bias + col0 + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 bv = __ldg(bp + i);
                v[4 * i] += bv.x; v[4 * i + 1] += bv.y; v[4 * i + 2] += bv.z; v[4 * i + 3] += bv.w;
              }
            }
          }
          epi_compute<EPI>(e, tc.z0, m, tc.n0 + (cbase + c) * 32, v, a0, a1, o0, o1, o2);
          // the stores that last used these output boxes must have finished reading them
          constexpr int OB = epi_out_bufs(EPI);
          const int ob = (OB == 2) ? buf : 0;
          if (lane == 0) {
            if (OB == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
          if (io & IO_OUT0) box_write_row(out_box + (0 * OB + ob) * EPI_BOX_BYTES, lane, o0);
          if (io & IO_OUT1) box_write_row(out_box + (1 * OB + ob) * EPI_BOX_BYTES, lane, o1);
          if constexpr (EPI == EPI_RELU) {
            if (io & IO_OUT2) box_write_row(out_box + (2 * OB + ob) * EPI_BOX_BYTES, lane, o2);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (g.l2_hints) {
              if (io & IO_OUT0)
                tma_store_2d_hint(&em.out0, out_box + (0 * OB + ob) * EPI_BOX_BYTES, col0 + c * 32, row0, stream_policy);
              if (io & IO_OUT1)
                tma_store_2d_hint(&em.out1, out_box + (1 * OB + ob) * EPI_BOX_BYTES, col1 + c * 32, row0, stream_policy);
              if constexpr (EPI == EPI_RELU) {
                if (io & IO_OUT2)
                  tma_store_2d_hint(&em.out1, out_box + (2 * OB + ob) * EPI_BOX_BYTES,
                                    col1 + c * 32 + static_cast<int>(e.o1_imag), row0, stream_policy);
              }
            } else {
              if (io & IO_OUT0)
                tma_store_2d(&em.out0, out_box + (0 * OB + ob) * EPI_BOX_BYTES, col0 + c * 32, row0);
              if (io & IO_OUT1)
                tma_store_2d(&em.out1, out_box + (1 * OB + ob) * EPI_BOX_BYTES, col1 + c * 32, row0);
              if constexpr (EPI == EPI_RELU) {
                if (io & IO_OUT2)
                  tma_store_2d(&em.out1, out_box + (2 * OB + ob) * EPI_BOX_BYTES,
                               col1 + c * 32 + static_cast<int>(e.o1_imag), row0);
              }
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (!ok) break;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        t = t_next;
        tc = tc_next;
      }
      if (lane == 0) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        if (*abort_flag && has_in && issued > gchunk) {
          // an input load may still be in flight: let it land (bounded)
          const uint32_t pending = issued - 1;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&ibar[pending & 1], (pending >> 1) & 1)) break;
        }
      }
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
