// Two chained bf16 GEMMs in one persistent sm_100a kernel: the [tokens, neurons] intermediate of a
// BDH layer is produced, transformed and consumed on chip.
//
//   Y   = A1 . B1^T                       (128 tokens x 128 neurons per chunk, K1 = D or T)
//   P   = epilogue(Y, aux inputs)         (gate / gate backward / rotation backward: gemm_sm100.cuh)
//   OUT += P . B2                         (128 tokens x N2 = D, contraction over the neurons)
//
// Y lives in TMEM, the epilogue warps turn it into the bf16 tile P, written straight into shared
// memory in the K-major 128-byte-swizzled layout that tcgen05.mma reads as its A operand; the same
// shared-memory tile is what TMA stores to global memory when the backward pass needs P. OUT stays
// in TMEM over all neuron chunks of an output tile. The three uses (reference: src/model/bdh.rs:359-441
// and its backward):
//   forward    Y = LN(a) E_v^T,  P = relu(Y) * x (dropout),          OUT = P . Dec     (the MLP output)
//   backward 1 Y = dmlp Dec^T,   P = dy (and the gate gradient dxg),  OUT = dy . E_v    (d LN(a), per head)
//   backward 2 Y = Gs q,         P = dx (rotation undone, + dxg),     OUT = dx . E      (d cur)
// so the [tokens, H*N] tensors x*y, dy and dx are written once and never read back by the GEMM that
// contracts them over the neurons.
//
// Work split: the (m-tile, neuron chunk) units are numbered with the chunk index fastest and cut
// into gridDim.x contiguous ranges, one per CTA, so every SM gets the same amount of work whatever
// the tile counts are. An output tile whose chunks are shared by several CTAs is written as fp32
// partial tiles (slot = CTA, running group index), which partials_reduce_kernel adds up in a fixed
// order: no atomics, no zero-fill, deterministic sums.
//
// Every [128 x 128] bf16 tile that crosses HBM moves by TMA: the auxiliary inputs (x, x*y, the gate
// gradient, the rotary table) land in shared-memory tiles two units ahead of their use, the epilogue
// warps transform them IN PLACE into the outputs (x -> x*y, x -> dy, x*y -> gate gradient, ...), and
// the same tiles are the second GEMM's A operand and the source of the global stores.
//
// Warp roles (384 threads): warp 0 feeds both operand rings by TMA; warp 1 issues the first GEMM's
// tcgen05.mma stream and warp 11 the second GEMM's (two issuers, because one thread's instruction
// rate is what bounds a kernel with this many short stages); warps 2-9 epilogue; warp 10 loads
// auxiliary tiles and stores finished ones. TMEM: two Y accumulators of 128 columns and one OUT
// accumulator of up to 256.
#pragma once
#include "gemm_sm100.cuh"

namespace bdh {

constexpr int DUAL_BM = 128;
constexpr int DUAL_BN1 = 128;        // neurons per chunk
constexpr int DUAL_BK = 64;
constexpr int DUAL_EW = 8;
constexpr int DUAL_THREADS = 32 * (2 + DUAL_EW + 2);
constexpr int DUAL_MAX_N2 = 256;
constexpr int DUAL_TILE_BYTES = DUAL_BM * DUAL_BN1 * 2;   // one [128 x 128] bf16 tile: two [128 x 64] swizzled boxes

struct DualArgs {
  int n_mt;             // 128-row token tiles
  int H, cph;           // heads; 128-neuron chunks per head
  int n_per_head;       // neurons per head (cph * 128)
  int K1;               // contraction length of the first GEMM (multiple of 64)
  int N2;               // output width (multiple of 64, <= 256)
  int group_per_head;   // 0: one output tile per m-tile (sum over all heads); 1: one per (m-tile, head)
  int tpb;              // m-tiles per sequence (T / 128)
  long long a1_b, a1_h; // A1 row of (m-tile, head) = (mt / tpb) * a1_b + (mt % tpb) * 128 + h * a1_h
  long long b1_b;       // MN-major B1: first k row of m-tile mt = (mt / tpb) * b1_b
  float* partials;      // [gridDim.x * maxg][128][N2] fp32
  int maxg;             // partial tiles per CTA
  EpiParams epi;        // alpha, theta, flags, dropout
  int* status;
  unsigned long long* trace;   // developer aid (null: off): CTA 0 stamps %globaltimer per unit and event, [unit][8]
};

struct DualUnit {
  int mt, h, nc;
  int grp;
  int a1_row, col, b1_k0;
};

// Walks the units of a CTA in order. The position is kept as (sequence, tile in sequence, head, chunk) counters
// that advance by increments: the single threads that issue TMA and MMA instructions run this once per unit, and
// a 64-bit division there costs more than the instructions they issue.
struct DualCursor {
  int b, tt, h, nc;
  __device__ __forceinline__ void seek(const DualArgs& g, long long u) {
    const int cpm = g.H * g.cph;
    const int mt = static_cast<int>(u / cpm);
    const int c = static_cast<int>(u - static_cast<long long>(mt) * cpm);
    h = c / g.cph;
    nc = c - h * g.cph;
    b = mt / g.tpb;
    tt = mt - b * g.tpb;
  }
  __device__ __forceinline__ void advance(const DualArgs& g) {
    if (++nc == g.cph) {
      nc = 0;
      if (++h == g.H) {
        h = 0;
        if (++tt == g.tpb) {
          tt = 0;
          ++b;
        }
      }
    }
  }
  __device__ __forceinline__ int mt(const DualArgs& g) const { return b * g.tpb + tt; }
  __device__ __forceinline__ int grp(const DualArgs& g) const { return g.group_per_head ? mt(g) * g.H + h : mt(g); }
  __device__ __forceinline__ int a1_row(const DualArgs& g) const {
    return static_cast<int>(b * g.a1_b + static_cast<long long>(tt) * DUAL_BM + h * g.a1_h);
  }
  __device__ __forceinline__ DualUnit unit(const DualArgs& g) const {
    DualUnit t;
    t.mt = mt(g);
    t.h = h;
    t.nc = nc;
    t.grp = grp(g);
    t.a1_row = a1_row(g);
    t.col = h * g.n_per_head + nc * DUAL_BN1;
    t.b1_k0 = static_cast<int>(b * g.b1_b);
    return t;
  }
};

// Event slots of the per-unit timeline that CTA 0 records when DualArgs::trace is set.
enum : int { TR_LOAD_ISSUED = 0, TR_IN_READY = 1, TR_Y_READY = 2, TR_P_WRITTEN = 3, TR_MMA2_FIRST = 4, TR_MMA2_LAST = 5,
             TR_SLOT_FREED = 6, TR_MMA1_FIRST = 7 };
constexpr int DUAL_TRACE_UNITS = 512;
__device__ __forceinline__ void dual_stamp(const DualArgs& g, long long unit, int ev) {
  if (g.trace && blockIdx.x == 0 && unit < DUAL_TRACE_UNITS) g.trace[unit * 16 + ev] = global_timer_ns();
}

// Units [lo, hi) of CTA `cta` out of `ctas`.
__host__ __device__ __forceinline__ long long dual_range_lo(long long total, int cta, int ctas) {
  return total * cta / ctas;
}

// Shared-memory plan. NTB = tile buffers per unit in flight (two units are in flight):
//   NTB = 1  one auxiliary input (x), transformed in place into P: 2 tiles; with a resident A1 the B1 and B2 rings
//            have three 16 KB stages each, else a 3-stage (A1, B1) ring and B2 in two stages of 64 neurons;
//   NTB = 2  two auxiliary tensors per unit (x and x*y -> dy and the gate gradient, or the gate gradient and the
//            rotary table): 4 tiles, a 2-stage (A1, B1) ring, B2 in two stages of 32 neurons. These kernels are
//            bound by their four [tokens, neurons] streams, so the shallower operand rings are not what limits them.
template <int NTB, int A1R>
struct DualSmem {
  // A1R = 1: the [128 x K1 <= 256] A1 tile of the current (m-tile, head) stays in shared memory for all of its
  // neuron chunks (it is the same for every chunk) and the first ring carries B1 alone: per 128 x 128 unit the SM
  // pulls 64 KB less through its L2 port, which is what bounds these kernels (K1 = D is short, so every chunk's
  // work needs its own 64 KB + 64 KB of weights).
  static constexpr int A1_RES_BYTES = A1R ? DUAL_BM * 256 * 2 : 0;                 // 64 KB
  static constexpr int R1 = A1R ? 3 : ((NTB == 1) ? 3 : 2);
  static constexpr int R2 = A1R ? 3 : 2;
  static constexpr int BK2 = (A1R || NTB == 2) ? 32 : 64;
  static constexpr int A1_BYTES = A1R ? 0 : DUAL_BM * DUAL_BK * 2;                 // 16 KB per stage when streamed
  static constexpr int B1_BYTES = DUAL_BN1 * DUAL_BK * 2;                          // 16 KB
  static constexpr int STAGE1 = A1_BYTES + B1_BYTES;
  static constexpr int STAGE2 = BK2 * DUAL_MAX_N2 * 2;
  static constexpr int A1_RES = 0;
  static constexpr int RING1 = A1_RES + A1_RES_BYTES;
  static constexpr int RING2 = RING1 + R1 * STAGE1;
  static constexpr int TILES = RING2 + R2 * STAGE2;               // [2 slots][NTB] tiles of 32 KB
  static constexpr int BARS = TILES + 2 * NTB * DUAL_TILE_BYTES;
  static constexpr int NUM_BARS = 2 * R1 + 2 * R2 + 5 * 2 + 2 + 2 + 2;
  static constexpr int TOTAL = BARS + NUM_BARS * 8 + 16 + 1024;   // +1024: manual alignment slack
  static_assert(TOTAL <= 227 * 1024, "shared-memory plan exceeds the per-CTA limit");
};

// A [128 x 128] bf16 tile in shared memory is two [128 x 64] boxes in the K-major 128-byte-swizzled layout
// (what TMA writes and reads for such a box and what tcgen05.mma takes as an A operand): row r at r * 128
// bytes inside its box, 16-byte chunk c stored at position c ^ (r & 7).
__device__ __forceinline__ uint8_t* tile_row_chunk(uint8_t* tile, int row, int col) {
  return tile + (col >> 6) * (DUAL_BM * 128) + row * 128;
}
__device__ __forceinline__ void tile_write_row(uint8_t* tile, int row, int col, const float (&v)[32]) {
  uint8_t* sub = tile_row_chunk(tile, row, col);
  const int c0 = (col & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u;
    u.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
    u.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
    u.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
    u.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(sub + (((c0 + j) ^ (row & 7)) << 4)) = u;
  }
}
__device__ __forceinline__ void tile_read_row(uint8_t* tile, int row, int col, uint32_t (&u)[16]) {
  const uint8_t* sub = tile_row_chunk(tile, row, col);
  const int c0 = (col & 63) >> 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 w = *reinterpret_cast<const uint4*>(sub + (((c0 + j) ^ (row & 7)) << 4));
    u[4 * j] = w.x; u[4 * j + 1] = w.y; u[4 * j + 2] = w.z; u[4 * j + 3] = w.w;
  }
}

struct DualMaps {
  CUtensorMap a1, b1, b2, p, in0, in1, out1;
};

template <int EPI, int B1_MN, int NTB, int A1R>
__global__ void __launch_bounds__(DUAL_THREADS, 1)
dual_gemm_kernel(const __grid_constant__ DualMaps tm, const DualArgs g) {
  using L = DualSmem<NTB, A1R>;
  constexpr int R1 = L::R1, R2 = L::R2, BK2 = L::BK2;
  constexpr int NKB2 = DUAL_BN1 / BK2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full1 = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t* empty1 = full1 + R1;
  uint64_t* full2 = empty1 + R1;
  uint64_t* empty2 = full2 + R2;
  uint64_t* yfull = empty2 + R2;          // [2] first-GEMM accumulator complete
  uint64_t* yempty = yfull + 2;           // [2] ... drained by the epilogue warps
  uint64_t* infull = yempty + 2;          // [2] auxiliary input tiles of the slot have landed
  uint64_t* a2full = infull + 2;          // [2] P (and the second output) written into the slot's tiles
  uint64_t* a2empty = a2full + 2;         // [2] slot consumed by the second GEMM and by the global stores
  uint64_t* obar = a2empty + 2;           // [0] output accumulator complete, [1] drained
  uint64_t* drain_bar = obar + 2;
  uint64_t* a1bar = drain_bar + 2;        // [0] resident A1 tile loaded, [1] its last consumer has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a1bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int IO_WARP = 2 + DUAL_EW;        // auxiliary tile loads + output tile stores
  constexpr int MMA2_WARP = IO_WARP + 1;      // second-GEMM issuer

  const EpiParams& e = g.epi;
  const int io = epi_io_mask(EPI, e.flags);
  const bool has_in0 = (io & IO_IN0) != 0, has_in1 = NTB == 2 && (io & IO_IN1) != 0;
  const bool has_out1 = NTB == 2 && EPI == EPI_GATE_BWD;

  if (threadIdx.x == 0) {
    for (int s = 0; s < R1; ++s) { mbar_init(&full1[s], 1); mbar_init(&empty1[s], 1); }
    for (int s = 0; s < R2; ++s) { mbar_init(&full2[s], 1); mbar_init(&empty2[s], 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&yfull[a], 1);
      mbar_init(&yempty[a], DUAL_EW);
      mbar_init(&infull[a], 1);
      mbar_init(&a2full[a], DUAL_EW);
      mbar_init(&a2empty[a], 2);
    }
    mbar_init(&obar[0], 1);
    mbar_init(&obar[1], DUAL_EW);
    mbar_init(&drain_bar[0], 1);
    mbar_init(&drain_bar[1], 1);
    mbar_init(&a1bar[0], 1);
    mbar_init(&a1bar[1], 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tm.a1);
    tma_prefetch_desc(&tm.b1);
    tma_prefetch_desc(&tm.b2);
    tma_prefetch_desc(&tm.p);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_out = tmem_base + 2 * DUAL_BN1;

  const long long total = static_cast<long long>(g.n_mt) * g.H * g.cph;
  const long long u_lo = dual_range_lo(total, blockIdx.x, gridDim.x);
  const long long u_hi = dual_range_lo(total, blockIdx.x + 1, gridDim.x);
  const long long n_units = u_hi - u_lo;
  const int nkb1 = g.K1 / DUAL_BK;
  const uint32_t stage2_bytes = static_cast<uint32_t>(BK2 * g.N2 * 2);
  auto tile_ptr = [&](int slot, int which) { return smem + L::TILES + (slot * NTB + which) * DUAL_TILE_BYTES; };

  if (warp == 0) {
    // ---------------- operand producer: the (A1, B1) ring (or the resident A1 tile + a B1 ring) and the B2 ring ----------------
    // One thread feeds both rings; each ring advances whenever its next stage is free (non-blocking tests), so
    // neither waits for the other.
    if (lane == 0) {
      const uint64_t keep = l2_policy_evict_last();     // weights and A1 rows are re-read by many CTAs
      int st1 = 0, st2 = 0;
      uint32_t ph1 = 0, ph2 = 0, armed1 = 0, par1 = 0, armed2 = 0, par2 = 0;
      long long u1 = 0, u2 = 0;                          // unit (relative) each ring is loading
      int kb1 = 0, kb2 = 0;
      DualCursor cu1, cu2;
      cu1.seek(g, u_lo);
      cu2.seek(g, u_lo);
      DualUnit t1 = cu1.unit(g), t2 = cu2.unit(g);
      int a1_cur = -1;
      uint32_t a1_loads = 0;
      uint32_t idle = 0;
      uint64_t t0 = 0;
      while (u1 < n_units || u2 < n_units) {
        bool progressed = false;
        if (u1 < n_units) {
          bool a1_ready = true;
          if (A1R && kb1 == 0 && t1.a1_row != a1_cur) {
            // a new (m-tile, head): replace the resident A1 tile once the MMAs that read the old one are done
            a1_ready = mbar_test_wait(&a1bar[1], (a1_loads & 1) ^ 1);
            if (a1_ready) {
              mbar_arrive_expect_tx(&a1bar[0], static_cast<uint32_t>(nkb1) * DUAL_BM * DUAL_BK * 2);
              for (int kb = 0; kb < nkb1; ++kb)
                tma_load_2d_hint(smem + L::A1_RES + kb * (DUAL_BM * DUAL_BK * 2), &tm.a1, &a1bar[0], kb * DUAL_BK,
                                 t1.a1_row, keep);
              a1_cur = t1.a1_row;
              ++a1_loads;
              progressed = true;
            }
          }
          if (a1_ready && mbar_test_wait(&empty1[st1], ph1 ^ 1)) {
            mbar_arrive_expect_tx(&full1[st1], L::STAGE1);
            armed1 |= 1u << st1;
            par1 = (par1 & ~(1u << st1)) | (ph1 << st1);
            uint8_t* sa = smem + L::RING1 + st1 * L::STAGE1;
            uint8_t* sb = sa + L::A1_BYTES;
            const int kc = kb1 * DUAL_BK;
            if (!A1R) tma_load_2d_hint(sa, &tm.a1, &full1[st1], kc, t1.a1_row, keep);
            if constexpr (B1_MN == 0) {
              tma_load_2d_hint(sb, &tm.b1, &full1[st1], kc, t1.col, keep);
            } else {
#pragma unroll
              for (int i = 0; i < DUAL_BN1 / 64; ++i)
                tma_load_2d_hint(sb + i * (DUAL_BK * 128), &tm.b1, &full1[st1], t1.col + i * 64, t1.b1_k0 + kc, keep);
            }
            if (++st1 == R1) { st1 = 0; ph1 ^= 1; }
            if (++kb1 == nkb1) {
              kb1 = 0;
              ++u1;
              cu1.advance(g);
              t1 = cu1.unit(g);
            }
            progressed = true;
          }
        }
        if (u2 < n_units && mbar_test_wait(&empty2[st2], ph2 ^ 1)) {
          mbar_arrive_expect_tx(&full2[st2], stage2_bytes);
          armed2 |= 1u << st2;
          par2 = (par2 & ~(1u << st2)) | (ph2 << st2);
          uint8_t* sb = smem + L::RING2 + st2 * L::STAGE2;
          // one 3-D box: N2/64 column groups of [BK2 neurons x 64 columns], laid out one after the other
          tma_load_3d_hint(sb, &tm.b2, &full2[st2], 0, t2.col + kb2 * BK2, 0, keep);
          if (++st2 == R2) { st2 = 0; ph2 ^= 1; }
          if (++kb2 == NKB2) {
            kb2 = 0;
            ++u2;
            cu2.advance(g);
            t2 = cu2.unit(g);
          }
          progressed = true;
        }
        if (progressed) {
          idle = 0;
          continue;
        }
        __nanosleep(20);
        if ((++idle & 255u) == 0) {
          if (idle == 256u) t0 = global_timer_ns();
          if (*abort_flag) break;
          if (global_timer_ns() - t0 > BDH_WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(g.status, STATUS_OK, STATUS_TIMEOUT_SMEM_EMPTY);
            break;
          }
        }
      }
      if (*abort_flag) {
        // let the copies that are still in flight land before the CTA's shared memory goes away
        for (int s = 0; s < R1; ++s) {
          if (!(armed1 & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&full1[s], (par1 >> s) & 1u)) break;
        }
        for (int s = 0; s < R2; ++s) {
          if (!(armed2 & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&full2[s], (par2 >> s) & 1u)) break;
        }
        if (A1R && a1_loads)
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&a1bar[0], (a1_loads - 1) & 1u)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- first-GEMM issuer: Y(i) = A1 . B1^T, one ring stage at a time ----------------
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(DUAL_BM, DUAL_BN1, 0, B1_MN);
      int s1 = 0;
      uint32_t ph1 = 0, a1_seen = 0;
      DualCursor c1;
      c1.seek(g, u_lo);
      int a1_have = -1;
      bool ok = true;
      for (long long i = 0; i < n_units && ok; ++i) {
        const int a = static_cast<int>(i & 1);
        const int a1_row = c1.a1_row(g);
        c1.advance(g);
        const int next_row = (i + 1 < n_units) ? c1.a1_row(g) : -1;
        if (!mbar_wait(&yempty[a], ((i >> 1) & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_EMPTY)) break;
        if (A1R && a1_row != a1_have) {
          if (!mbar_wait(&a1bar[0], a1_seen & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) break;
          a1_have = a1_row;
          ++a1_seen;
        }
        tc_fence_after();
        dual_stamp(g, i, TR_MMA1_FIRST);
        const uint32_t d_tmem = tmem_base + a * DUAL_BN1;
        for (int kb = 0; kb < nkb1; ++kb) {
          if (!mbar_wait(&full1[s1], ph1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + L::RING1 + s1 * L::STAGE1) + L::A1_BYTES;
          const uint32_t sa = A1R ? smem_u32(smem + L::A1_RES + kb * (DUAL_BM * DUAL_BK * 2)) : sb - L::A1_BYTES;
#pragma unroll
          for (int k = 0; k < DUAL_BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = (B1_MN == 0) ? make_smem_desc(sb + k * 32, 16, 1024)
                                             : make_smem_desc(sb + k * 2048, DUAL_BK * 128, 1024);
            umma_bf16(d_tmem, da, db, idesc1, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty1[s1]);
          if (++s1 == R1) { s1 = 0; ph1 ^= 1; }
        }
        if (!ok) break;
        umma_commit(&yfull[a]);
        // the A1 tile may be replaced once the last unit that reads it has been computed
        if (A1R && next_row != a1_row) umma_commit(&a1bar[1]);
      }
      if (*abort_flag) {
        umma_commit(&drain_bar[0]);
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(&drain_bar[0], 0)) break;
      }
    }
  } else if (warp == MMA2_WARP) {
    // ---------------- second-GEMM issuer: OUT += P(i) . B2, one B2 stage at a time ----------------
    if (lane == 0) {
      const uint32_t idesc2 = make_idesc_bf16(DUAL_BM, g.N2, 0, 1);
      int s2 = 0;
      uint32_t ph2 = 0, groups_done = 0;
      DualCursor c2;
      c2.seek(g, u_lo);
      int grp_prev = -1;
      bool ok = true;
      for (long long i = 0; i < n_units && ok; ++i) {
        const int slot = static_cast<int>(i & 1);
        const int grp = c2.grp(g);
        c2.advance(g);
        const bool first = grp != grp_prev;
        const bool last = (i + 1 == n_units) || (c2.grp(g) != grp);
        grp_prev = grp;
        if (!mbar_wait(&a2full[slot], (i >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) break;
        if (first && !mbar_wait(&obar[1], (groups_done & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        dual_stamp(g, i, TR_MMA2_FIRST);
        const uint32_t a2 = smem_u32(tile_ptr(slot, 0));
        for (int kb = 0; kb < NKB2; ++kb) {
          if (!mbar_wait(&full2[s2], ph2, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + L::RING2 + s2 * L::STAGE2);
#pragma unroll
          for (int k = 0; k < BK2 / 16; ++k) {
            const int kk = kb * (BK2 / 16) + k;             // 16-column step inside the 128-column P tile
            const uint64_t da = make_smem_desc(a2 + (kk >> 2) * (DUAL_BM * 128) + (kk & 3) * 32, 16, 1024);
            const uint64_t db = make_smem_desc(sb + k * 2048, BK2 * 128, 1024);
            umma_bf16(tmem_out, da, db, idesc2, (first && kk == 0) ? 0u : 1u);
          }
          umma_commit(&empty2[s2]);
          if (++s2 == R2) { s2 = 0; ph2 ^= 1; }
        }
        if (!ok) break;
        dual_stamp(g, i, TR_MMA2_LAST);
        umma_commit(&a2empty[slot]);
        if (last) {
          umma_commit(&obar[0]);
          ++groups_done;
        }
      }
      if (*abort_flag) {
        // let the MMAs already issued retire before TMEM is released
        umma_commit(&drain_bar[1]);
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(&drain_bar[1], 0)) break;
      }
    }
  } else if (warp == IO_WARP) {
    // ---------------- auxiliary input tiles in (two units ahead of their use), finished tiles out ----------------
    if (lane == 0) {
      uint32_t armed = 0, armed_parity = 0;
      const uint64_t stream = l2_policy_evict_first();  // [tokens, neurons] tiles pass through L2 once
      const uint64_t keep = l2_policy_evict_last();
      const uint32_t in_bytes = (has_in0 ? DUAL_TILE_BYTES : 0) + (has_in1 ? DUAL_TILE_BYTES : 0);
      DualCursor cl, cs;             // unit being loaded / unit being stored
      cl.seek(g, u_lo);
      cs.seek(g, u_lo);
      for (long long i = 0; i <= n_units; ++i) {
        if (i < n_units) {
          // the slot is free once the second GEMM of unit i-2 and the stores of its tiles are done with it
          const int slot = static_cast<int>(i & 1);
          if (!mbar_wait(&a2empty[slot], ((i >> 1) & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_EMPTY)) break;
          const DualUnit t = cl.unit(g);
          cl.advance(g);
          const int row = t.mt * DUAL_BM;
          dual_stamp(g, i, TR_LOAD_ISSUED);
          if (in_bytes) {
            mbar_arrive_expect_tx(&infull[slot], in_bytes);
            armed |= 1u << slot;
            armed_parity = (armed_parity & ~(1u << slot)) | (static_cast<uint32_t>((i >> 1) & 1) << slot);
          } else {
            mbar_arrive(&infull[slot]);
          }
          if (has_in0) {
            tma_load_3d_hint(tile_ptr(slot, 0), &tm.in0, &infull[slot], 0, row, t.col >> 6, stream);
          }
          if (has_in1) {
            // the rotary table is indexed by (position in the sequence, column inside the head)
            const int r1 = (EPI == EPI_DQ_BWD) ? (t.mt % g.tpb) * DUAL_BM : row;
            const int c1 = (EPI == EPI_DQ_BWD) ? t.nc * DUAL_BN1 : t.col;
            const uint64_t pol1 = (EPI == EPI_DQ_BWD) ? keep : stream;
            tma_load_3d_hint(tile_ptr(slot, NTB - 1), &tm.in1, &infull[slot], 0, r1, c1 >> 6, pol1);
          }
        }
        if (i > 0) {
          const int slot = static_cast<int>((i - 1) & 1);
          if (!mbar_wait(&a2full[slot], ((i - 1) >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) break;
          const DualUnit t = cs.unit(g);
          cs.advance(g);
          const int row = t.mt * DUAL_BM;
          tma_store_3d_hint(&tm.p, tile_ptr(slot, 0), 0, row, t.col >> 6, stream);
          if (has_out1) {
            tma_store_3d_hint(&tm.out1, tile_ptr(slot, NTB - 1), 0, row, t.col >> 6, stream);
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          // the stores have finished reading shared memory: the tiles may be overwritten
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          dual_stamp(g, i - 1, TR_SLOT_FREED);
          mbar_arrive(&a2empty[slot]);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (*abort_flag) {
        for (int s = 0; s < 2; ++s) {
          if (!(armed & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&infull[s], (armed_parity >> s) & 1u)) break;
        }
      }
    }
  } else {
    // ---------------- epilogue: Y (TMEM) + auxiliary tiles (shared memory) -> P in place ; OUT (TMEM) -> fp32 partial tile ----------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // which 64 of the chunk's 128 columns
    const int trow = q * 32 + lane;         // row inside the 128-row tile
    uint32_t groups_done = 0;
    DualCursor cur;
    cur.seek(g, u_lo);
    DualUnit t = cur.unit(g);
    for (long long i = 0; i < n_units; ++i) {
      const int a = static_cast<int>(i & 1);
      const bool more = i + 1 < n_units;
      cur.advance(g);
      const DualUnit tn = cur.unit(g);
      if (!mbar_wait(&infull[a], (i >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) break;
      if (threadIdx.x == 64) dual_stamp(g, i, TR_IN_READY);
      if (!mbar_wait(&yfull[a], (i >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL)) break;
      if (threadIdx.x == 64) dual_stamp(g, i, TR_Y_READY);
      tc_fence_after();
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * DUAL_BN1;
      uint8_t* tile0 = tile_ptr(a, 0);
      uint8_t* tile1 = tile_ptr(a, NTB - 1);
      const int m = t.mt * DUAL_BM + trow;
      {
        // both 32-column halves of this warp's share are fetched from TMEM before any arithmetic, so the two
        // loads' latencies overlap
        float v0[32], v1[32];
        const int c0 = half * 64, c1 = half * 64 + 32;   // columns inside the chunk
        tmem_ld_32x32(tacc + c0, v0);
        tmem_ld_32x32(tacc + c1, v1);
        tmem_ld_wait();
        auto finish = [&](int ccol, float (&v)[32]) {
          float o0[32], o1[32], o2[32];
          uint32_t r0[16], r1[16];
          if (has_in0) tile_read_row(tile0, trow, ccol, r0);
          if (has_in1) tile_read_row(tile1, trow, ccol, r1);
          epi_compute<EPI>(e, t.h, m, t.nc * DUAL_BN1 + ccol, v, r0, r1, o0, o1, o2);
          if constexpr (EPI == EPI_RELU_GATE) {
            tile_write_row(tile0, trow, ccol, o1);           // P = x*y
          } else {
            tile_write_row(tile0, trow, ccol, o0);           // P = dy (gate backward) or dx (rotation backward)
            if constexpr (EPI == EPI_GATE_BWD) tile_write_row(tile1, trow, ccol, o1);
          }
        };
        finish(c0, v0);
        finish(c1, v1);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&yempty[a]);
        mbar_arrive(&a2full[a]);
        if (warp == 2) dual_stamp(g, i, TR_P_WRITTEN);
      }
      const bool last = !more || tn.grp != t.grp;
      if (last) {
        // the output tile is complete for this CTA's share of the chunks: write it as an fp32 partial tile
        if (!mbar_wait(&obar[0], groups_done & 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
        float* part = g.partials +
                      (static_cast<long long>(blockIdx.x) * g.maxg + groups_done) * DUAL_BM * g.N2 +
                      static_cast<long long>(trow) * g.N2;
        const uint32_t tout = tmem_out + (static_cast<uint32_t>(q * 32) << 16);
        const int c_lo = half * (g.N2 / 2), c_hi = c_lo + g.N2 / 2;
        for (int c = c_lo; c < c_hi; c += 32) {
          float v[32];
          tmem_ld_32x32(tout + c, v);
          tmem_ld_wait();
          float4* p4 = reinterpret_cast<float4*>(part + c);
#pragma unroll
          for (int j = 0; j < 8; ++j) p4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&obar[1]);
        ++groups_done;
      }
      t = tn;
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

// OUT tile of group `grp` = sum, in CTA order, of the partial tiles written by the CTAs whose unit
// range touches the group. One warp per output row, 8 columns per lane and step.
//   out row of (group, r) = (grp % heads_out) * out_h_stride + (grp / heads_out) * 128 + r
// with heads_out = H for per-head groups (head-major output [H * M, N2]) and 1 otherwise.
template <bool OUT_BF16, bool ACCUM>
__global__ void partials_reduce_kernel(const float* __restrict__ partials, void* __restrict__ out, long long total_units,
                                       int units_per_group, int producer_ctas, int maxg, int N2, long long n_groups,
                                       int heads_out, long long out_h_stride, long long ld_out) {
  const long long row_id = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long grp = row_id / DUAL_BM;
  if (grp >= n_groups) return;
  const int r = static_cast<int>(row_id - grp * DUAL_BM);
  const int lane = threadIdx.x & 31;
  const long long g_lo = grp * units_per_group, g_hi = g_lo + units_per_group;
  // first CTA whose range ends after g_lo
  int cta = static_cast<int>(g_lo * producer_ctas / total_units);
  while (cta + 1 < producer_ctas && dual_range_lo(total_units, cta + 1, producer_ctas) <= g_lo) ++cta;
  while (cta > 0 && dual_range_lo(total_units, cta, producer_ctas) > g_lo) --cta;
  const long long orow = (grp % heads_out) * out_h_stride + (grp / heads_out) * DUAL_BM + r;
  for (int c = lane * 8; c < N2; c += 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = cta; k < producer_ctas; ++k) {
      const long long lo = dual_range_lo(total_units, k, producer_ctas);
      const long long hi = dual_range_lo(total_units, k + 1, producer_ctas);
      if (lo >= g_hi) break;
      if (hi <= g_lo || hi <= lo) continue;
      const long long local = grp - lo / units_per_group;      // running group index inside CTA k
      const float4* p = reinterpret_cast<const float4*>(
          partials + ((static_cast<long long>(k) * maxg + local) * DUAL_BM + r) * N2 + c);
      const float4 u0 = p[0], u1 = p[1];
      acc[0] += u0.x; acc[1] += u0.y; acc[2] += u0.z; acc[3] += u0.w;
      acc[4] += u1.x; acc[5] += u1.y; acc[6] += u1.z; acc[7] += u1.w;
    }
    if (OUT_BF16) {
      uint4 u;
      u.x = pack_bf16x2(acc[0], acc[1]); u.y = pack_bf16x2(acc[2], acc[3]);
      u.z = pack_bf16x2(acc[4], acc[5]); u.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(out) + orow * ld_out + c) = u;
    } else {
      float4* o = reinterpret_cast<float4*>(static_cast<float*>(out) + orow * ld_out + c);
      float4 a0 = make_float4(acc[0], acc[1], acc[2], acc[3]), a1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (ACCUM) {
        const float4 p0 = o[0], p1 = o[1];
        a0.x += p0.x; a0.y += p0.y; a0.z += p0.z; a0.w += p0.w;
        a1.x += p1.x; a1.y += p1.y; a1.z += p1.z; a1.w += p1.w;
      }
      o[0] = a0;
      o[1] = a1;
    }
  }
}

}  // namespace bdh
