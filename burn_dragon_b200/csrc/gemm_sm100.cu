// Host side of the tcgen05 GEMM: builds the TMA descriptors for both operands and launches the
// persistent kernel instantiation that matches (operand majors, epilogue).
#include "bdh_kernels.h"
#include "gemm_sm100.cuh"

#include <mutex>

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
  return r == CUDA_SUCCESS ? BDH_OK : BDH_ERR_TMAP;
}

static int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, int A_MN, int B_MN, int EPI>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int max_ctas,
                  cudaStream_t stream) {
  constexpr int STAGES = (BN == 256) ? 4 : 6;
  using L = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, EPI, STAGES>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
        cudaSuccess)
      return BDH_ERR_LAUNCH;
    configured = true;
  }
  const long long tiles_m = (g.M + GEMM_BM - 1) / GEMM_BM;
  const long long tiles_n = (g.N + BN - 1) / BN;
  long long tiles = tiles_m * tiles_n * g.nz0 * g.nz1;
  int grid = static_cast<int>(tiles < max_ctas ? tiles : max_ctas);
  if (grid < 1) grid = 1;
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

}  // namespace bdh

using namespace bdh;

extern "C" int bdh_gemm_bf16(const BdhMat* A, int a_mn, const BdhMat* B, int b_mn,
                             const BdhGemmDesc* d, cudaStream_t stream) {
  if (d->M <= 0 || d->N <= 0 || d->K <= 0 || d->nz0 <= 0 || d->nz1 <= 0) return BDH_ERR_ARGUMENT;
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

  const int max_ctas = d->max_ctas > 0 ? d->max_ctas : num_sms();
  const int key = (a_mn ? 1 : 0) | (b_mn ? 2 : 0);

#define BDH_CASE(BN_, AMN, BMN, EPI_)                                                 \
  if (bn == BN_ && key == ((AMN) | ((BMN) << 1)) && d->epi == EPI_)                   \
    return launch<BN_, AMN, BMN, EPI_>(ta, tb, g, max_ctas, stream);

  BDH_CASE(256, 0, 0, EPI_STORE)
  BDH_CASE(256, 0, 0, EPI_RELU)
  BDH_CASE(256, 0, 0, EPI_RELU_GATE)
  BDH_CASE(256, 0, 0, EPI_CAUSAL)
  BDH_CASE(256, 0, 0, EPI_GATE_BWD)
  BDH_CASE(256, 0, 1, EPI_STORE)
  BDH_CASE(256, 0, 1, EPI_DQ_BWD)
  BDH_CASE(256, 1, 1, EPI_STORE)
  BDH_CASE(256, 1, 0, EPI_STORE)
  BDH_CASE(128, 0, 0, EPI_STORE)
  BDH_CASE(128, 0, 0, EPI_CAUSAL)
  BDH_CASE(128, 0, 1, EPI_STORE)
  BDH_CASE(128, 1, 1, EPI_STORE)
#undef BDH_CASE
  return BDH_ERR_UNSUPPORTED;
}
