// Host side of the chained-GEMM kernel (dual_gemm_sm100.cuh): tensor maps, work split, launch, and
// the reduction of the fp32 partial tiles.
#include "bdh_kernels.h"
#include "device_once.h"
#include "dual_gemm_sm100.cuh"

#include <mutex>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <vector>

namespace bdh {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn dual_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 row-major matrix -> tensor map with a 128-byte-swizzled box of 64 columns x box_rows.
static int dual_tmap(CUtensorMap* out, const BdhMat& m, int box_rows) {
  EncodeTiledFn enc = dual_encode_fn();
  if (!enc) return BDH_ERR_DRIVER;
  if (!m.ptr || (reinterpret_cast<uintptr_t>(m.ptr) & 15) || (m.ld % 8) != 0) return BDH_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(m.cols), static_cast<cuuint64_t>(m.rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(m.ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(m.ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BDH_OK : BDH_ERR_TMAP;
}

// Row-major bf16 matrix seen as (64 columns, rows, 64-column groups): one box = `groups` adjacent
// [box_rows x 64] boxes, each 128-byte swizzled, stored one after the other in shared memory.
static int dual_tmap3(CUtensorMap* out, const BdhMat& m, int box_rows, int groups) {
  EncodeTiledFn enc = dual_encode_fn();
  if (!enc) return BDH_ERR_DRIVER;
  if (!m.ptr || (reinterpret_cast<uintptr_t>(m.ptr) & 15) || (m.ld % 8) != 0 || (m.cols % 64) != 0) return BDH_ERR_ALIGNMENT;
  cuuint64_t dims[3] = {64u, static_cast<cuuint64_t>(m.rows), static_cast<cuuint64_t>(m.cols / 64)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(m.ld) * 2, 128u};
  cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(groups)};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(m.ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BDH_OK : BDH_ERR_TMAP;
}

template <int EPI, int B1_MN, int NTB, int A1R>
static int dual_launch(const DualMaps& tm, const DualArgs& g, int grid, cudaStream_t stream) {
  using L = DualSmem<NTB, A1R>;
  auto kern = dual_gemm_kernel<EPI, B1_MN, NTB, A1R>;
  static PerDeviceOnce configured;
  if (configured.run([&] {
        return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) == cudaSuccess
                   ? 0 : 1;
      }))
    return BDH_ERR_LAUNCH;
  kern<<<grid, DUAL_THREADS, L::TOTAL, stream>>>(tm, g);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// Developer aid: with BDH_DUAL_TRACE=<file> in the environment every launch is followed by a device
// synchronisation and CTA 0's per-unit event stamps (%globaltimer, ns) are appended to <file> as text.
static unsigned long long* dual_trace_buffer() {
  static unsigned long long* buf = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    if (getenv("BDH_DUAL_TRACE")) {
      if (cudaMalloc(&buf, sizeof(unsigned long long) * 16 * DUAL_TRACE_UNITS) != cudaSuccess) buf = nullptr;
    }
  }
  return buf;
}

static void dual_trace_dump(unsigned long long* buf, int epi, cudaStream_t stream) {
  cudaStreamSynchronize(stream);
  std::vector<unsigned long long> h(16 * DUAL_TRACE_UNITS);
  cudaMemcpy(h.data(), buf, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  FILE* f = fopen(getenv("BDH_DUAL_TRACE"), "a");
  if (!f) return;
  fprintf(f, "# epi %d: unit load_issued in_ready y_ready p_written mma2_first mma2_last slot_freed mma1_first (ns from first stamp)\n", epi);
  unsigned long long t0 = ~0ull;
  for (size_t i = 0; i < h.size(); ++i) if ((i % 16) < 8 && h[i] && h[i] < t0) t0 = h[i];
  for (int u = 0; u < DUAL_TRACE_UNITS; ++u) {
    if (!h[u * 16 + TR_P_WRITTEN]) break;
    fprintf(f, "%d", u);
    for (int k = 0; k < 8; ++k) fprintf(f, " %lld", h[u * 16 + k] ? (long long)(h[u * 16 + k] - t0) : -1ll);
    for (int k = 8; k < 11; ++k) fprintf(f, " %lld", (long long)h[u * 16 + k]);
    fprintf(f, "\n");
  }
  fclose(f);
}

static int dual_grid(const BdhDualDesc* d, long long total) {
  int ctas = d->max_ctas > 0 ? d->max_ctas : current_device_sms();
  if (ctas > total) ctas = static_cast<int>(total);
  return ctas < 1 ? 1 : ctas;
}

static int dual_maxg(long long total, int ctas, int units_per_group) {
  const long long per_cta = (total + ctas - 1) / ctas;
  return static_cast<int>((per_cta + units_per_group - 1) / units_per_group) + 1;
}

}  // namespace bdh

using namespace bdh;

extern "C" long long bdh_dual_gemm_partial_floats(const BdhDualDesc* d) {
  if (d->M <= 0 || d->H <= 0 || d->n_per_head <= 0 || d->N2 <= 0) return 0;
  const long long total = static_cast<long long>(d->M / DUAL_BM) * d->H * (d->n_per_head / DUAL_BN1);
  if (total <= 0) return 0;
  const int ctas = dual_grid(d, total);
  const int upg = (d->n_per_head / DUAL_BN1) * (d->group_per_head ? 1 : d->H);
  return static_cast<long long>(ctas) * dual_maxg(total, ctas, upg) * DUAL_BM * d->N2;
}

extern "C" int bdh_dual_gemm(const BdhMat* A1, const BdhMat* B1, int b1_mn, const BdhMat* B2, const BdhMat* P,
                             const BdhDualDesc* d, cudaStream_t stream) {
  if (d->M <= 0 || (d->M % DUAL_BM) || d->H <= 0 || d->n_per_head <= 0 || (d->n_per_head % DUAL_BN1) || d->K1 <= 0 ||
      (d->K1 % DUAL_BK) || d->N2 <= 0 || (d->N2 % 64) || d->N2 > DUAL_MAX_N2 || d->T <= 0 || (d->T % DUAL_BM) ||
      (d->M % d->T) || !d->partials)
    return BDH_ERR_ARGUMENT;
  bind_primary_context();
  const int epi = d->epi;
  if (epi != EPI_RELU_GATE && epi != EPI_GATE_BWD && epi != EPI_DQ_BWD) return BDH_ERR_UNSUPPORTED;
  const int io = epi_io_mask(epi, d->flags | (epi == EPI_RELU_GATE ? EPI_F_NO_OUT0 : 0));
  // auxiliary tensors are read / written 16 bytes at a time per row
  auto bad = [](const void* p, long long ld) { return !p || (reinterpret_cast<uintptr_t>(p) & 15) || (ld % 8); };
  if ((io & IO_IN0) && bad(d->in0, d->ld_in0)) return BDH_ERR_ALIGNMENT;
  if ((io & IO_IN1) && bad(d->in1, d->ld_in1)) return BDH_ERR_ALIGNMENT;
  if (epi == EPI_GATE_BWD && bad(d->out1, d->ld_out1)) return BDH_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(d->partials) & 15)) return BDH_ERR_ALIGNMENT;
  if (epi == EPI_DQ_BWD && (d->flags & EPI_F_ROPE) && !(d->flags & EPI_F_TABLE)) return BDH_ERR_UNSUPPORTED;
  if (d->flags & EPI_F_POPE) return BDH_ERR_UNSUPPORTED;

  // tiles per unit in flight: the forward gate has one auxiliary tensor (x, turned into x*y in place), the two
  // backward kernels have two
  const int ntb = epi == EPI_RELU_GATE ? 1 : 2;
  const long long HN = static_cast<long long>(d->H) * d->n_per_head;
  DualMaps tm;
  memset(&tm, 0, sizeof(tm));
  int rc = dual_tmap(&tm.a1, *A1, DUAL_BM);
  if (rc) return rc;
  rc = dual_tmap(&tm.b1, *B1, b1_mn ? DUAL_BK : DUAL_BN1);
  if (rc) return rc;
  // the forward gate keeps its A1 tile (LN(a) rows of one head, K1 = D <= 256) resident in shared memory
  const int a1r = (epi == EPI_RELU_GATE && d->K1 <= 256) ? 1 : 0;
  {
    // B2 [neurons, >= N2 columns]: a stage is BK2 neurons x N2 columns
    const BdhMat b2v{B2->ptr, B2->rows, d->N2, B2->ld};
    rc = dual_tmap3(&tm.b2, b2v, a1r ? DualSmem<1, 1>::BK2 : (ntb == 1 ? DualSmem<1, 0>::BK2 : DualSmem<2, 0>::BK2), d->N2 / 64);
  }
  if (rc) return rc;
  {
    const BdhMat pv{P->ptr, P->rows, HN, P->ld};
    rc = dual_tmap3(&tm.p, pv, DUAL_BM, 2);
  }
  if (rc) return rc;
  if (io & IO_IN0) {
    const BdhMat m{d->in0, d->M, HN, d->ld_in0};
    if ((rc = dual_tmap3(&tm.in0, m, DUAL_BM, 2))) return rc;
  }
  if (io & IO_IN1) {
    const bool table = epi == EPI_DQ_BWD;
    const BdhMat m{d->in1, table ? d->T : d->M, table ? d->n_per_head : HN, d->ld_in1};
    if ((rc = dual_tmap3(&tm.in1, m, DUAL_BM, 2))) return rc;
  }
  if (epi == EPI_GATE_BWD) {
    const BdhMat m{d->out1, d->M, HN, d->ld_out1};
    if ((rc = dual_tmap3(&tm.out1, m, DUAL_BM, 2))) return rc;
  }

  DualArgs g;
  memset(&g, 0, sizeof(g));
  g.n_mt = d->M / DUAL_BM;
  g.H = d->H;
  g.n_per_head = d->n_per_head;
  g.cph = d->n_per_head / DUAL_BN1;
  g.K1 = d->K1;
  g.N2 = d->N2;
  g.group_per_head = d->group_per_head ? 1 : 0;
  g.tpb = d->T / DUAL_BM;
  g.a1_b = d->a1_b;
  g.a1_h = d->a1_h;
  g.b1_b = d->b1_b;
  g.partials = d->partials;
  g.status = d->status;
  EpiParams& e = g.epi;
  e.alpha = d->alpha; e.theta = d->theta;
  e.T = d->T; e.pos0 = d->pos0;
  e.n_per_head = d->n_per_head;
  e.freqs = nullptr; e.slopes = nullptr; e.bias = nullptr;
  e.flags = d->flags | (epi == EPI_RELU_GATE ? EPI_F_NO_OUT0 : 0);
  e.drop_p = d->drop_p; e.drop_seed = d->drop_seed;

  g.trace = dual_trace_buffer();
  if (g.trace) cudaMemsetAsync(g.trace, 0, sizeof(unsigned long long) * 16 * DUAL_TRACE_UNITS, stream);
  const long long total = static_cast<long long>(g.n_mt) * g.H * g.cph;
  const int ctas = dual_grid(d, total);
  g.maxg = dual_maxg(total, ctas, g.cph * (g.group_per_head ? 1 : g.H));
  if (d->partial_floats < static_cast<long long>(ctas) * g.maxg * DUAL_BM * g.N2) return BDH_ERR_TOO_LARGE;

#define BDH_DUAL_CASE(EPI_, BMN, NTB_, A1R_)                                        \
  if (epi == EPI_ && (b1_mn ? 1 : 0) == BMN && a1r == A1R_) {                       \
    rc = dual_launch<EPI_, BMN, NTB_, A1R_>(tm, g, ctas, stream);                   \
    if (g.trace && rc == BDH_OK) dual_trace_dump(g.trace, epi, stream);             \
    return rc;                                                                      \
  }
  BDH_DUAL_CASE(EPI_RELU_GATE, 0, 1, 1)
  BDH_DUAL_CASE(EPI_RELU_GATE, 0, 1, 0)
  BDH_DUAL_CASE(EPI_GATE_BWD, 0, 2, 0)
  BDH_DUAL_CASE(EPI_DQ_BWD, 1, 2, 0)
#undef BDH_DUAL_CASE
  return BDH_ERR_UNSUPPORTED;
}

extern "C" int bdh_dual_gemm_reduce(const BdhDualDesc* d, void* out, long long ld_out, int out_bf16, int accumulate,
                                    long long out_h_stride, cudaStream_t stream) {
  if (d->M <= 0 || (d->M % DUAL_BM) || (d->n_per_head % DUAL_BN1) || (d->N2 % 8) || !out || !d->partials ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out % 8))
    return BDH_ERR_ARGUMENT;
  const int cph = d->n_per_head / DUAL_BN1;
  const long long n_mt = d->M / DUAL_BM;
  const long long total = n_mt * d->H * cph;
  const int ctas = dual_grid(d, total);
  const int upg = cph * (d->group_per_head ? 1 : d->H);
  const int maxg = dual_maxg(total, ctas, upg);
  const long long n_groups = n_mt * (d->group_per_head ? d->H : 1);
  const int heads_out = d->group_per_head ? d->H : 1;
  const long long rows = n_groups * DUAL_BM;
  const int rows_per_block = 8;
  const unsigned grid = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
  if (out_bf16)
    partials_reduce_kernel<true, false><<<grid, 32 * rows_per_block, 0, stream>>>(
        d->partials, out, total, upg, ctas, maxg, d->N2, n_groups, heads_out, out_h_stride, ld_out);
  else if (accumulate)
    partials_reduce_kernel<false, true><<<grid, 32 * rows_per_block, 0, stream>>>(
        d->partials, out, total, upg, ctas, maxg, d->N2, n_groups, heads_out, out_h_stride, ld_out);
  else
    partials_reduce_kernel<false, false><<<grid, 32 * rows_per_block, 0, stream>>>(
        d->partials, out, total, upg, ctas, maxg, d->N2, n_groups, heads_out, out_h_stride, ld_out);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}
