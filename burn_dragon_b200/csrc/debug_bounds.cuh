// Checked build (-DBDH_DEBUG_BOUNDS): every index that comes out of DATA (a token id, a target id, a
// column block of a sparse pattern) is compared with its extent before it is used. The first
// violation of a translation unit is written to a device record {site, index, extent, where}; the
// kernel then carries on with its normal defensive behaviour (clamp, ignore, zero-fill), so a checked
// run never traps and never touches memory the unchecked run would not touch. The host reads the
// record after the step (`torch.ops.bdh.bounds_records()`); a clean run reads site 0.
//
// Indices that come out of loop bounds are not instrumented: they are covered by running every kernel
// on tiny and non-multiple-of-tile shapes against the fp32 statements in the GPU tests.
#pragma once
#include <cuda_runtime.h>

namespace bdh {

enum BoundsSite : int {
  BOUNDS_OK = 0,
  BOUNDS_EMBED_TOKEN = 1,       // embed_ln_fwd: token id outside [0, vocab)
  BOUNDS_EMBED_BWD_TOKEN = 2,   // embed_ln_bwd: the same ids on the way back
  BOUNDS_CE_TARGET = 3,         // cross_entropy: target outside [0, vocab) and not the ignore value -100
  BOUNDS_GRAPH_COLUMN = 4,      // graph_spmm_relu: column block outside [0, ceil(D / 64))
};

#ifdef BDH_DEBUG_BOUNDS
struct BoundsRecord {
  int site;
  int pad;
  long long index, extent, where;
};
static __device__ BoundsRecord g_bounds_record;      // one per translation unit

__device__ __forceinline__ void bounds_check(long long index, long long extent, int site, long long where) {
  if (index >= 0 && index < extent) return;
  if (atomicCAS(&g_bounds_record.site, BOUNDS_OK, site) == BOUNDS_OK) {
    g_bounds_record.index = index;
    g_bounds_record.extent = extent;
    g_bounds_record.where = where;
  }
}
#define BDH_BOUNDS_CHECK(index, extent, site, where) ::bdh::bounds_check((index), (extent), (site), (where))

// out: {1, site, index, extent, where}; `clear` resets the record after reading it.
static inline int bounds_record_read(long long out[5], int clear) {
  BoundsRecord r{};
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&r, g_bounds_record, sizeof(r)) != cudaSuccess) return -1;
  out[0] = 1; out[1] = r.site; out[2] = r.index; out[3] = r.extent; out[4] = r.where;
  if (clear) {
    BoundsRecord zero{};
    if (cudaMemcpyToSymbol(g_bounds_record, &zero, sizeof(zero)) != cudaSuccess) return -1;
  }
  return 0;
}
#else
#define BDH_BOUNDS_CHECK(index, extent, site, where) ((void)0)
// out: {0, 0, 0, 0, 0}: this library was built without the checks.
static inline int bounds_record_read(long long out[5], int) {
  for (int i = 0; i < 5; ++i) out[i] = 0;
  return 0;
}
#endif

}  // namespace bdh
