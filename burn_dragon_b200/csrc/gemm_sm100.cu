// Host side of the tcgen05 GEMM: builds the TMA descriptors for both operands and launches the
// persistent kernel instantiation that matches (operand majors, epilogue).
#include <cstdlib>
#include "bdh_kernels.h"
#include "gemm_sm100.cuh"
#include "device_once.h"

#include <mutex>
#include <stdio.h>
#include <string.h>

namespace bdh {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 row-major matrix -> tensor map with a 128-byte-swizzled box of 64 columns x box_rows.
static int make_tmap(CUtensorMap* out, const BdhMat& m, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return BDH_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(m.ptr) & 15) || (m.ld % 8) != 0) return BDH_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(m.cols), static_cast<cuuint64_t>(m.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(m.ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(m.ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "bdh gemm: tensor map rejected (driver code %d): ptr %p rows %lld cols %lld ld %lld box rows %d\n",
            static_cast<int>(r), m.ptr, m.rows, m.cols, m.ld, box_rows);
  return r == CUDA_SUCCESS ? BDH_OK : BDH_ERR_TMAP;
}

// bf16 output / auxiliary-input tensor -> tensor map with 32 x 32 boxes and the 64-byte swizzle.
static int make_epi_tmap(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return BDH_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {32u, 32u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BDH_OK : BDH_ERR_TMAP;
}

static int num_sms() { return current_device_sms(); }

template <int BN, int A_MN, int B_MN, int EPI, bool TMA_EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const EpiMaps& em, const GemmArgs& g,
                  int max_ctas, cudaStream_t stream) {
  // Staged epilogues run 8 epilogue warps; the mainloop ring gets what shared memory is left.
  constexpr int EW = TMA_EPI ? 8 : 4;
  constexpr int STAGE_BYTES = (GEMM_BM + BN) * GEMM_BK * 2;
  constexpr int EPI_BYTES = TMA_EPI ? EW * (2 * epi_num_in(EPI) + epi_out_bufs(EPI) * epi_num_out(EPI)) * EPI_BOX_BYTES
                                    : (EPI == EPI_STORE ? EW * EPI_RED_TILE_BYTES : 0);
  constexpr int BUDGET = 227 * 1024 - 2048 - EPI_BYTES;
  constexpr int FIT = BUDGET / STAGE_BYTES;
  constexpr int STAGES = FIT > 6 ? 6 : FIT;
  static_assert(STAGES >= 2, "not enough shared memory for the mainloop ring");
  using L = GemmSmem<BN, STAGES, TMA_EPI, EW, EPI>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI, STAGES, TMA_EPI, EW>;
  static PerDeviceOnce configured;   // the shared-memory limit is a per-device attribute
  if (configured.run([&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) == cudaSuccess ? 0 : 1;
      }))
    return BDH_ERR_LAUNCH;
  const long long tiles_m = (g.M + GEMM_BM - 1) / GEMM_BM;
  const long long tiles_n = (g.N + BN - 1) / BN;
  long long tiles = tiles_m * tiles_n * g.nz0 * g.nz1;
  int grid = static_cast<int>(tiles < max_ctas ? tiles : max_ctas);
  if (grid < 1) grid = 1;
  if (g.gather.world > 1) {
    GemmArgs gg = g;
    gg.gather.target = EW;          // every epilogue warp of the copying CTA counts a finished block once
    kern<<<grid, gemm_threads(EW), L::TOTAL, stream>>>(ta, tb, em, gg);
    return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
  }
  kern<<<grid, gemm_threads(EW), L::TOTAL, stream>>>(ta, tb, em, g);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

}  // namespace bdh

using namespace bdh;

extern "C" int bdh_gemm_bf16(const BdhMat* A, int a_mn, const BdhMat* B, int b_mn,
                             const BdhGemmDesc* d, cudaStream_t stream) {
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->nz0 <= 0 || d->nz1 <= 0) return BDH_ERR_ARGUMENT;
  bind_primary_context();
  const int bn = d->bn == 128 ? 128 : 256;
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, *A, a_mn ? GEMM_BK : GEMM_BM);
  if (rc) return rc;
  rc = make_tmap(&tb, *B, b_mn ? GEMM_BK : bn);
  if (rc) return rc;

  GemmArgs g;
  g.M = d->M; g.N = d->N; g.K = d->K;
  g.nz0 = d->nz0; g.nz1 = d->nz1;
  g.a = {d->a_off[0], d->a_off[1], d->a_off[2], d->a_off[3]};
  g.b = {d->b_off[0], d->b_off[1], d->b_off[2], d->b_off[3]};
  g.causal_tiles = d->causal_tiles;
  g.causal_k = d->causal_k;
  g.tile_shift = 0;
  g.tile_skip = (d->epi == EPI_CAUSAL) ? d->tile_skip : nullptr;
  {
    // BDH_GEMM_L2_HINTS=1 launches with the L2 eviction hints (read once per process). Off by default: measured
    // on the layer kernels at 8 sequences, the hints left the encoder unchanged (0.177 ms) and slowed the gate
    // kernels (y-gate 0.134 -> 0.150 ms, gate backward 0.195 -> 0.217 ms); the training step did not move.
    static const int hints = [] { const char* v = getenv("BDH_GEMM_L2_HINTS"); return (v && v[0] == '1') ? 1 : 0; }();
    g.l2_hints = hints;
  }
  g.status = d->status;
  EpiParams& e = g.epi;
  e.out0 = d->out0; e.out1 = d->out1; e.in0 = d->in0; e.in1 = d->in1;
  e.ld_out0 = d->ld_out0; e.ld_out1 = d->ld_out1; e.ld_in0 = d->ld_in0; e.ld_in1 = d->ld_in1;
  e.c_m0 = d->c_off[0]; e.c_m1 = d->c_off[1]; e.c_n0 = d->c_off[2]; e.c_n1 = d->c_off[3];
  e.o1_n0 = d->o1_off[0]; e.o1_n1 = d->o1_off[1]; e.o1_imag = d->o1_off[2];
  e.alpha = d->alpha; e.theta = d->theta;
  e.T = d->T > 0 ? d->T : 1; e.pos0 = d->pos0;
  e.n_per_head = d->n_per_head > 0 ? d->n_per_head : 1;
  e.freqs = d->freqs; e.slopes = d->slopes; e.flags = d->flags;
  e.bias = d->bias;
  if (d->bias && (reinterpret_cast<uintptr_t>(d->bias) & 15)) return BDH_ERR_ALIGNMENT;
  e.drop_p = d->drop_p; e.drop_seed = d->drop_seed;
  e.peer_rows = d->peer_rows > 0 ? d->peer_rows : 1;
  e.peer_world = d->peer_world;
  e.peer_rank = d->peer_rank;
  for (int i = 0; i < GEMM_MAX_PEERS; ++i)
    e.peer_out[i] = (d->peer_out && i < d->peer_world) ? reinterpret_cast<float*>(d->peer_out[i]) : nullptr;
  if (d->flags & EPI_F_PEER_RS) {
    if (d->epi != EPI_STORE || !d->peer_out || d->peer_world < 1 || d->peer_world > GEMM_MAX_PEERS ||
        d->peer_rows < 1 || d->peer_rank < 0 || d->peer_rank >= d->peer_world)
      return BDH_ERR_ARGUMENT;
    if (d->causal_tiles == 0) {
      // Tiles are walked with z1 slowest, then z0, then rows. One pass over all owners takes `cycle`
      // consecutive tiles; rank r starts r/world of a cycle ahead, so at any moment the ranks store
      // into different owners instead of all into the same one.
      const long long per_z = ((d->M + GEMM_BM - 1) / GEMM_BM) * ((d->N + bn - 1) / bn);
      const long long total = per_z * d->nz0 * d->nz1;
      const long long cycle = (d->c_off[0] >= d->c_off[1] || d->nz1 == 1) ? per_z * d->nz0 : total;
      g.tile_shift = static_cast<int>((d->peer_rank * (cycle / d->peer_world)) % total);
    }
  }

  memset(&g.gather, 0, sizeof(g.gather));
  if (d->gather_world > 1) {
    if (a_mn || d->nz0 != 1 || d->nz1 != 1 || d->gather_world > GEMM_MAX_PEERS || !d->gather_src || !d->gather_arrived ||
        d->gather_rank < 0 || d->gather_rank >= d->gather_world || d->gather_rows < GEMM_BM || (d->gather_rows % GEMM_BM) ||
        d->gather_rows * d->gather_world != d->M || A->ld != d->K || (d->K % 8) || d->causal_tiles || d->causal_k ||
        (d->flags & EPI_F_PEER_RS))
      return BDH_ERR_ARGUMENT;
    GatherArgs& ga = g.gather;
    for (int i = 0; i < GEMM_MAX_PEERS; ++i)
      ga.src[i] = i < d->gather_world ? reinterpret_cast<const uint4*>(d->gather_src[i]) : nullptr;
    ga.dst = reinterpret_cast<uint4*>(const_cast<void*>(A->ptr));
    ga.block_vec = static_cast<long long>(GEMM_BM) * d->K * 2 / 16;
    ga.blocks_per_shard = static_cast<int>(d->gather_rows / GEMM_BM);
    ga.arrived = d->gather_arrived;
    ga.target = 0;                  // set by launch() to the instantiation's number of epilogue warps
    ga.world = d->gather_world;
    ga.rank = d->gather_rank;
    // walk the tiles from this rank's own rows on, then the next rank's, ... (the order the blocks arrive in)
    const long long tiles_n = (d->N + bn - 1) / bn;
    g.tile_shift = static_cast<int>(static_cast<long long>(ga.rank) * ga.blocks_per_shard * tiles_n);
  }

  const int max_ctas = d->max_ctas > 0 ? d->max_ctas : num_sms();
  const int key = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);

  // Decide whether the outputs / auxiliary inputs can move through the staged TMA epilogue.
  EpiMaps em;
  memset(&em, 0, sizeof(em));
  bool tma_epi = !d->no_tma_epilogue && epi_tma_capable(d->epi, d->flags);
  const int io = epi_io_mask(d->epi, d->flags);
  const bool batched = d->nz0 * d->nz1 > 1;
  if (batched && ((d->M % GEMM_BM) || (d->N % bn))) tma_epi = false;
  for (int i = 0; i < 4; ++i) if (d->c_off[i] % 8) tma_epi = false;
  if (d->bias && (d->N % 32)) tma_epi = false;      // the staged epilogue reads the bias 16 bytes at a time
  if (d->o1_off[0] % 8 || d->o1_off[1] % 8 || d->o1_off[2] % 8) tma_epi = false;
  if (tma_epi) {
    const long long rows = d->c_off[0] * (d->nz0 - 1) + d->c_off[1] * (d->nz1 - 1) + d->M;
    const long long cols = d->c_off[2] * (d->nz0 - 1) + d->c_off[3] * (d->nz1 - 1) + d->N;
    const long long cols1 = (d->epi == EPI_RELU)
                                ? d->o1_off[0] * (d->nz0 - 1) + d->o1_off[1] * (d->nz1 - 1) + d->N +
                                      ((d->flags & EPI_F_POPE) ? d->o1_off[2] : 0)
                                : cols;
    // the rotary table (in0 of EPI_RELU, in1 of EPI_DQ_BWD) is a [T, n_per_head] tensor of its own
    const bool tab0 = d->epi == EPI_RELU, tab1 = d->epi == EPI_DQ_BWD;
    if ((io & (tab0 ? IO_IN0 : 0)) || (io & (tab1 ? IO_IN1 : 0)))
      if ((e.T % 32) || (e.n_per_head % 32)) tma_epi = false;
    struct { int bit; const void* p; long long ld; long long rows; long long cols; CUtensorMap* m; } t[4] = {
        {IO_OUT0, d->out0, d->ld_out0, rows, cols, &em.out0},
        {IO_OUT1, d->out1, d->ld_out1, rows, cols1, &em.out1},
        {IO_IN0, d->in0, d->ld_in0, tab0 ? e.T : rows, tab0 ? e.n_per_head : cols, &em.in0},
        {IO_IN1, d->in1, d->ld_in1, tab1 ? e.T : rows, tab1 ? e.n_per_head : cols, &em.in1}};
    for (auto& x : t) {
      if (!tma_epi) break;
      if (!(io & x.bit)) continue;
      if (!x.p || (reinterpret_cast<uintptr_t>(x.p) & 15) || (x.ld % 8) ||
          make_epi_tmap(x.m, x.p, x.rows, x.cols, x.ld) != BDH_OK) {
        tma_epi = false;
        break;
      }
    }
  }

#define BDH_CASE(BN_, AMN, BMN, EPI_)                                                   \
  if (bn == BN_ && key == ((AMN) | ((BMN) << 1)) && d->epi == EPI_) {                   \
    if (tma_epi) return launch<BN_, AMN, BMN, EPI_, true>(ta, tb, em, g, max_ctas, stream); \
    return launch<BN_, AMN, BMN, EPI_, false>(ta, tb, em, g, max_ctas, stream);           \
  }

  BDH_CASE(256, 0, 0, EPI_STORE)
  BDH_CASE(256, 0, 0, EPI_RELU)
  BDH_CASE(256, 0, 0, EPI_RELU_GATE)
  BDH_CASE(256, 0, 0, EPI_CAUSAL)
  BDH_CASE(256, 0, 0, EPI_GATE_BWD)
  BDH_CASE(256, 0, 1, EPI_STORE)
  BDH_CASE(256, 0, 1, EPI_DQ_BWD)
  BDH_CASE(256, 0, 0, EPI_DQ_BWD)      // (state terms of the chunked attention: both operands K-major)
  BDH_CASE(256, 1, 1, EPI_STORE)
  BDH_CASE(256, 1, 0, EPI_STORE)
  BDH_CASE(128, 0, 0, EPI_STORE)
  BDH_CASE(128, 0, 0, EPI_CAUSAL)
  BDH_CASE(128, 0, 1, EPI_STORE)
  BDH_CASE(128, 1, 1, EPI_STORE)
#undef BDH_CASE
  return BDH_ERR_UNSUPPORTED;
}
