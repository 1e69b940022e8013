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
// Warp roles (352 threads): warp 0 TMA producer of the (A1, B1) ring; warp 1 issues every
// tcgen05.mma; warps 2-9 epilogue; warp 10 loads the B2 ring and stores finished P tiles.
// TMEM: two Y accumulators of 128 columns and one OUT accumulator of up to 256 columns.
#pragma once
#include "gemm_sm100.cuh"

namespace bdh {

constexpr int DUAL_BM = 128;
constexpr int DUAL_BN1 = 128;        // neurons per chunk
constexpr int DUAL_BK = 64;
constexpr int DUAL_EW = 8;
constexpr int DUAL_THREADS = 32 * (2 + DUAL_EW + 1);
constexpr int DUAL_R1 = 3;           // (A1, B1) ring stages of 64 k-columns
constexpr int DUAL_R2 = 2;           // B2 ring stages of 64 neurons x N2
constexpr int DUAL_MAX_N2 = 256;

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
  EpiParams epi;        // in0 / in1 / out1 with leading dimensions, alpha, theta, flags, dropout, rotary
  int* status;
};

struct DualUnit {
  int mt, h, nc;
  long long grp;
  int a1_row, col, b1_k0;
};

__device__ __forceinline__ DualUnit dual_decode(const DualArgs& g, long long u) {
  DualUnit t;
  const int cpm = g.H * g.cph;
  t.mt = static_cast<int>(u / cpm);
  const int c = static_cast<int>(u - static_cast<long long>(t.mt) * cpm);
  t.h = c / g.cph;
  t.nc = c - t.h * g.cph;
  t.grp = g.group_per_head ? static_cast<long long>(t.mt) * g.H + t.h : t.mt;
  const int b = t.mt / g.tpb;
  t.a1_row = static_cast<int>(b * g.a1_b + static_cast<long long>(t.mt - b * g.tpb) * DUAL_BM + t.h * g.a1_h);
  t.col = t.h * g.n_per_head + t.nc * DUAL_BN1;
  t.b1_k0 = static_cast<int>(b * g.b1_b);
  return t;
}

// Units [lo, hi) of CTA `cta` out of `ctas`.
__host__ __device__ __forceinline__ long long dual_range_lo(long long total, int cta, int ctas) {
  return total * cta / ctas;
}

struct DualSmem {
  static constexpr int A1_BYTES = DUAL_BM * DUAL_BK * 2;          // 16 KB
  static constexpr int B1_BYTES = DUAL_BN1 * DUAL_BK * 2;         // 16 KB
  static constexpr int STAGE1 = A1_BYTES + B1_BYTES;
  static constexpr int STAGE2 = DUAL_BK * DUAL_MAX_N2 * 2;        // 32 KB
  static constexpr int A2_BYTES = DUAL_BM * DUAL_BN1 * 2;         // 32 KB: two [128 x 64] K-major sub-tiles
  static constexpr int RING1 = 0;
  static constexpr int RING2 = RING1 + DUAL_R1 * STAGE1;
  static constexpr int A2 = RING2 + DUAL_R2 * STAGE2;
  static constexpr int BARS = A2 + 2 * A2_BYTES;
  static constexpr int NUM_BARS = 2 * DUAL_R1 + 2 * DUAL_R2 + 2 + 2 + 2 + 2 + 2 + 1;
  static constexpr int TOTAL = BARS + NUM_BARS * 8 + 16 + 1024;   // +1024: manual alignment slack
};

// Packed bf16 row of 32 values -> the P tile in shared memory (K-major, 128-byte swizzle: row r at
// r * 128 bytes inside its [128 x 64] sub-tile, 16-byte chunk c stored at position c ^ (r & 7)).
__device__ __forceinline__ void a2_write_row(uint8_t* a2, int row, int col, const float (&v)[32]) {
  uint8_t* sub = a2 + (col >> 6) * (DUAL_BM * 128) + row * 128;
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

// 32 consecutive bf16 (64 bytes, 16-byte aligned) of one row, streamed past L1.
__device__ __forceinline__ void dual_load_32(const void* base, long long ld, long long r, long long c,
                                             uint32_t (&u)[16]) {
  const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + r * ld + c);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 w;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                 : "l"(p + i));
    u[4 * i] = w.x; u[4 * i + 1] = w.y; u[4 * i + 2] = w.z; u[4 * i + 3] = w.w;
  }
}

template <int EPI, int B1_MN>
__global__ void __launch_bounds__(DUAL_THREADS, 1)
dual_gemm_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                 const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmP,
                 const DualArgs g) {
  using L = DualSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full1 = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t* empty1 = full1 + DUAL_R1;
  uint64_t* full2 = empty1 + DUAL_R1;
  uint64_t* empty2 = full2 + DUAL_R2;
  uint64_t* yfull = empty2 + DUAL_R2;     // [2] first-GEMM accumulator complete
  uint64_t* yempty = yfull + 2;           // [2] ... drained by the epilogue warps
  uint64_t* a2full = yempty + 2;          // [2] P tile written
  uint64_t* a2empty = a2full + 2;         // [2] P tile consumed by the second GEMM and by its global store
  uint64_t* obar = a2empty + 2;           // [0] output accumulator complete, [1] drained
  uint64_t* drain_bar = obar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int AUX_WARP = 2 + DUAL_EW;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DUAL_R1; ++s) { mbar_init(&full1[s], 1); mbar_init(&empty1[s], 1); }
    for (int s = 0; s < DUAL_R2; ++s) { mbar_init(&full2[s], 1); mbar_init(&empty2[s], 1); }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&yfull[a], 1);
      mbar_init(&yempty[a], DUAL_EW);
      mbar_init(&a2full[a], DUAL_EW);
      mbar_init(&a2empty[a], 2);
    }
    mbar_init(&obar[0], 1);
    mbar_init(&obar[1], DUAL_EW);
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA1);
    tma_prefetch_desc(&tmB1);
    tma_prefetch_desc(&tmB2);
    tma_prefetch_desc(&tmP);
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
  const int nkb1 = g.K1 / DUAL_BK;
  const uint32_t stage2_bytes = static_cast<uint32_t>(DUAL_BK * g.N2 * 2);

  if (warp == 0) {
    // ---------------- (A1, B1) ring producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      for (long long u = u_lo; u < u_hi && ok; ++u) {
        const DualUnit t = dual_decode(g, u);
        for (int kb = 0; kb < nkb1; ++kb) {
          if (!mbar_wait(&empty1[stage], phase ^ 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full1[stage], L::STAGE1);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          uint8_t* sa = smem + L::RING1 + stage * L::STAGE1;
          uint8_t* sb = sa + L::A1_BYTES;
          const int kc = kb * DUAL_BK;
          tma_load_2d(sa, &tmA1, &full1[stage], kc, t.a1_row);
          if constexpr (B1_MN == 0) {
            tma_load_2d(sb, &tmB1, &full1[stage], kc, t.col);
          } else {
#pragma unroll
            for (int i = 0; i < DUAL_BN1 / 64; ++i)
              tma_load_2d(sb + i * (DUAL_BK * 128), &tmB1, &full1[stage], t.col + i * 64, t.b1_k0 + kc);
          }
          if (++stage == DUAL_R1) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        for (int s = 0; s < DUAL_R1; ++s) {
          if (!(armed & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&full1[s], (armed_parity >> s) & 1u)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: Y(i+1) is issued before OUT += P(i) so that the tensor pipe works on
    // the next chunk's first GEMM while the epilogue warps turn chunk i's Y into P ----------------
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(DUAL_BM, DUAL_BN1, 0, B1_MN);
      const uint32_t idesc2 = make_idesc_bf16(DUAL_BM, g.N2, 0, 1);
      int s1 = 0, s2 = 0;
      uint32_t ph1 = 0, ph2 = 0;
      uint32_t groups_done = 0;
      bool ok = true;
      auto mma1 = [&](long long i) {   // i = unit index relative to u_lo
        const int a = static_cast<int>(i & 1);
        if (!mbar_wait(&yempty[a], ((i >> 1) & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * DUAL_BN1;
        for (int kb = 0; kb < nkb1; ++kb) {
          if (!mbar_wait(&full1[s1], ph1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) return false;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + L::RING1 + s1 * L::STAGE1);
          const uint32_t sb = sa + L::A1_BYTES;
#pragma unroll
          for (int k = 0; k < DUAL_BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = (B1_MN == 0) ? make_smem_desc(sb + k * 32, 16, 1024)
                                             : make_smem_desc(sb + k * 2048, DUAL_BK * 128, 1024);
            umma_bf16(d_tmem, da, db, idesc1, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty1[s1]);
          if (++s1 == DUAL_R1) { s1 = 0; ph1 ^= 1; }
        }
        umma_commit(&yfull[a]);
        return true;
      };
      const long long n_units = u_hi - u_lo;
      if (n_units > 0) ok = mma1(0);
      for (long long i = 0; i < n_units && ok; ++i) {
        if (i + 1 < n_units && !mma1(i + 1)) { ok = false; break; }
        const DualUnit t = dual_decode(g, u_lo + i);
        const bool first = (i == 0) || (dual_decode(g, u_lo + i - 1).grp != t.grp);
        const bool last = (i + 1 == n_units) || (dual_decode(g, u_lo + i + 1).grp != t.grp);
        const int b = static_cast<int>(i & 1);
        if (!mbar_wait(&a2full[b], (i >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
        if (first && !mbar_wait(&obar[1], (groups_done & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a2 = smem_u32(smem + L::A2 + b * L::A2_BYTES);
        for (int kb = 0; kb < DUAL_BN1 / DUAL_BK && ok; ++kb) {
          if (!mbar_wait(&full2[s2], ph2, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + L::RING2 + s2 * L::STAGE2);
#pragma unroll
          for (int k = 0; k < DUAL_BK / 16; ++k) {
            const uint64_t da = make_smem_desc(a2 + kb * (DUAL_BM * 128) + k * 32, 16, 1024);
            const uint64_t db = make_smem_desc(sb + k * 2048, DUAL_BK * 128, 1024);
            umma_bf16(tmem_out, da, db, idesc2, (first && kb == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&empty2[s2]);
          if (++s2 == DUAL_R2) { s2 = 0; ph2 ^= 1; }
        }
        if (!ok) break;
        umma_commit(&a2empty[b]);
        if (last) {
          umma_commit(&obar[0]);
          ++groups_done;
        }
      }
      if (*abort_flag) {
        umma_commit(drain_bar);
        for (int it = 0; it < (1 << 16); ++it)
          if (mbar_try_wait(drain_bar, 0)) break;
      }
    }
  } else if (warp == AUX_WARP) {
    // ---------------- B2 ring producer + global store of finished P tiles ----------------
    if (lane == 0) {
      int s2 = 0;
      uint32_t ph2 = 0, armed = 0, armed_parity = 0;
      bool ok = true;
      const long long n_units = u_hi - u_lo;
      for (long long i = 0; i <= n_units && ok; ++i) {
        bool stored = false;
        if (i > 0) {
          // P tile of unit i-1: two [128 x 64] boxes, as soon as the epilogue warps have written it
          const int b = static_cast<int>((i - 1) & 1);
          if (!mbar_wait(&a2full[b], ((i - 1) >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_FULL)) break;
          const DualUnit t = dual_decode(g, u_lo + i - 1);
          const uint8_t* a2 = smem + L::A2 + b * L::A2_BYTES;
          tma_store_2d(&tmP, a2, t.col, t.mt * DUAL_BM);
          tma_store_2d(&tmP, a2 + DUAL_BM * 128, t.col + 64, t.mt * DUAL_BM);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          stored = true;
        }
        if (i < n_units) {
          const DualUnit t = dual_decode(g, u_lo + i);
          for (int kb = 0; kb < DUAL_BN1 / DUAL_BK; ++kb) {
            if (!mbar_wait(&empty2[s2], ph2 ^ 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_EMPTY)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full2[s2], stage2_bytes);
            armed |= 1u << s2;
            armed_parity = (armed_parity & ~(1u << s2)) | (ph2 << s2);
            uint8_t* sb = smem + L::RING2 + s2 * L::STAGE2;
            for (int j = 0; j < g.N2 / 64; ++j)
              tma_load_2d(sb + j * (DUAL_BK * 128), &tmB2, &full2[s2], j * 64, t.col + kb * DUAL_BK);
            if (++s2 == DUAL_R2) { s2 = 0; ph2 ^= 1; }
          }
        }
        if (stored) {
          // the store has finished reading shared memory: the tile may be overwritten
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          mbar_arrive(&a2empty[(i - 1) & 1]);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (*abort_flag) {
        for (int s = 0; s < DUAL_R2; ++s) {
          if (!(armed & (1u << s))) continue;
          for (int it = 0; it < (1 << 16); ++it)
            if (mbar_try_wait(&full2[s], (armed_parity >> s) & 1u)) break;
        }
      }
    }
  } else {
    // ---------------- epilogue: Y (TMEM) -> P (shared memory, bf16) ; OUT (TMEM) -> fp32 partial tile ----------------
    const EpiParams& e = g.epi;
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // which 64 of the chunk's 128 columns
    const int io = epi_io_mask(EPI, e.flags);
    const int trow = q * 32 + lane;         // row inside the 128-row tile
    const long long n_units = u_hi - u_lo;
    const bool table_in1 = (EPI == EPI_DQ_BWD);
    uint32_t r0a[16], r1a[16], r0b[16], r1b[16];
    uint32_t groups_done = 0;
    typedef __nv_bfloat16 bf;

    auto load_in = [&](const DualUnit& t, int sub, uint32_t (&r0)[16], uint32_t (&r1)[16]) {
      const long long row = static_cast<long long>(t.mt) * DUAL_BM + trow;
      const long long col = t.col + half * 64 + sub * 32;
      if (io & IO_IN0) dual_load_32(e.in0, e.ld_in0, row, col, r0);
      if (io & IO_IN1) {
        if (table_in1)
          dual_load_32(e.in1, e.ld_in1, row % e.T, t.nc * DUAL_BN1 + half * 64 + sub * 32, r1);
        else
          dual_load_32(e.in1, e.ld_in1, row, col, r1);
      }
    };
    auto process = [&](const DualUnit& t, int sub, uint32_t tacc, uint8_t* a2, const uint32_t (&r0)[16],
                       const uint32_t (&r1)[16]) {
      float v[32], o0[32], o1[32], o2[32];
      const int ccol = half * 64 + sub * 32;             // column inside the chunk
      tmem_ld_32x32(tacc + ccol, v);
      tmem_ld_wait();
      const int m = t.mt * DUAL_BM + trow;
      epi_compute<EPI>(e, t.h, m, t.nc * DUAL_BN1 + ccol, v, r0, r1, o0, o1, o2);
      if constexpr (EPI == EPI_RELU_GATE) {
        a2_write_row(a2, trow, ccol, o1);                // P = x*y
      } else {
        a2_write_row(a2, trow, ccol, o0);                // P = dy (gate backward) or dx (rotation backward)
        if constexpr (EPI == EPI_GATE_BWD)
          store_bf16_32(static_cast<bf*>(e.out1), e.ld_out1, m, t.col + ccol, o1, 32);
      }
    };

    DualUnit t{};
    if (n_units > 0) {
      t = dual_decode(g, u_lo);
      load_in(t, 0, r0a, r1a);
    }
    bool ok = true;
    for (long long i = 0; i < n_units && ok; ++i) {
      const int a = static_cast<int>(i & 1);
      const bool more = i + 1 < n_units;
      DualUnit tn = t;
      if (more) tn = dual_decode(g, u_lo + i + 1);
      load_in(t, 1, r0b, r1b);
      if (!mbar_wait(&yfull[a], (i >> 1) & 1, abort_flag, g.status, STATUS_TIMEOUT_TMEM_FULL)) break;
      if (!mbar_wait(&a2empty[a], ((i >> 1) & 1) ^ 1, abort_flag, g.status, STATUS_TIMEOUT_SMEM_EMPTY)) break;
      tc_fence_after();
      const uint32_t tacc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * DUAL_BN1;
      uint8_t* a2 = smem + L::A2 + a * L::A2_BYTES;
      process(t, 0, tacc, a2, r0a, r1a);
      if (more) load_in(tn, 0, r0a, r1a);
      process(t, 1, tacc, a2, r0b, r1b);
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&yempty[a]);
        mbar_arrive(&a2full[a]);
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
