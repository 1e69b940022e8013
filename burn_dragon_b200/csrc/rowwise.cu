// Row-wise kernels of the BDH layer: affine-free LayerNorm (eps 1e-5, biased variance; reference
// src/model/bdh.rs:86-89), the embedding gather fused with its LayerNorm (bdh.rs:319-320), the
// layer tail cur' = LN(cur + LN(mlp)) (bdh.rs:436-441), mean cross-entropy (src/model/loss.rs:5-18)
// and the AdamW update. One warp owns one row; a row of D bf16 values is held in registers as
// 16-byte vectors, so each row is read once and written once.
#include "bdh_kernels.h"
#include "sm100_ptx.cuh"
#include "debug_bounds.cuh"

namespace bdh {

constexpr int ROW_MAX_CHUNKS = 8;  // 8 chunks * 32 lanes * 8 elements = 2048 columns
constexpr float LN_EPS = 1e-5f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int NC>
struct Row {
  float v[NC][8];
};

template <int NC>
__device__ __forceinline__ void row_load_bf16(Row<NC>& r, const __nv_bfloat16* p, int D, int lane) {
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
    if (c < D) {
      uint4 u = *reinterpret_cast<const uint4*>(p + c);
      float2 f;
      f = unpack_bf16x2(u.x); r.v[j][0] = f.x; r.v[j][1] = f.y;
      f = unpack_bf16x2(u.y); r.v[j][2] = f.x; r.v[j][3] = f.y;
      f = unpack_bf16x2(u.z); r.v[j][4] = f.x; r.v[j][5] = f.y;
      f = unpack_bf16x2(u.w); r.v[j][6] = f.x; r.v[j][7] = f.y;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) r.v[j][i] = 0.f;
    }
  }
}
template <int NC>
__device__ __forceinline__ void row_load_f32(Row<NC>& r, const float* p, int D, int lane) {
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
    if (c < D) {
      float4 a = *reinterpret_cast<const float4*>(p + c);
      float4 b = *reinterpret_cast<const float4*>(p + c + 4);
      r.v[j][0] = a.x; r.v[j][1] = a.y; r.v[j][2] = a.z; r.v[j][3] = a.w;
      r.v[j][4] = b.x; r.v[j][5] = b.y; r.v[j][6] = b.z; r.v[j][7] = b.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) r.v[j][i] = 0.f;
    }
  }
}
template <int NC>
__device__ __forceinline__ void row_store_bf16(const Row<NC>& r, __nv_bfloat16* p, int D, int lane) {
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
    if (c < D) {
      uint4 u;
      u.x = pack_bf16x2(r.v[j][0], r.v[j][1]);
      u.y = pack_bf16x2(r.v[j][2], r.v[j][3]);
      u.z = pack_bf16x2(r.v[j][4], r.v[j][5]);
      u.w = pack_bf16x2(r.v[j][6], r.v[j][7]);
      *reinterpret_cast<uint4*>(p + c) = u;
    }
  }
}
template <int NC>
__device__ __forceinline__ void row_store_f32(const Row<NC>& r, float* p, int D, int lane, bool accum) {
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
    if (c < D) {
#pragma unroll
      for (int i = 0; i < 8; ++i) p[c + i] = accum ? p[c + i] + r.v[j][i] : r.v[j][i];
    }
  }
}

// In place: r <- (r - mean) * rstd. Columns >= D hold zeros and are restored to zero.
template <int NC>
__device__ __forceinline__ void row_layernorm(Row<NC>& r, int D, int lane) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) s += r.v[j][i];
  const float mean = warp_sum(s) / D;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float d = (c < D) ? r.v[j][i] - mean : 0.f;
      r.v[j][i] = d;
      q += d * d;
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / D + LN_EPS);
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) r.v[j][i] *= rstd;
}

// Given y = LN(x) in `y` (already normalised) and upstream grad in `dy`, overwrite dy with dx.
// rstd must be recomputed by the caller from x; here we take it as an argument.
template <int NC>
__device__ __forceinline__ void row_layernorm_bwd(const Row<NC>& y, Row<NC>& dy, float rstd, int D, int lane) {
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s1 += dy.v[j][i];
      s2 += dy.v[j][i] * y.v[j][i];
    }
  const float m1 = warp_sum(s1) / D, m2 = warp_sum(s2) / D;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      dy.v[j][i] = (c < D) ? rstd * (dy.v[j][i] - m1 - y.v[j][i] * m2) : 0.f;
  }
}

// LayerNorm that also returns rstd (needed by the backward).
template <int NC>
__device__ __forceinline__ float row_layernorm_rstd(Row<NC>& r, int D, int lane) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) s += r.v[j][i];
  const float mean = warp_sum(s) / D;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    int c = (j * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float d = (c < D) ? r.v[j][i] - mean : 0.f;
      r.v[j][i] = d;
      q += d * d;
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / D + LN_EPS);
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) r.v[j][i] *= rstd;
  return rstd;
}

constexpr int ROW_WARPS = 8;

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_fwd_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> r;
    row_load_bf16(r, x + row * D, D, lane);
    row_layernorm(r, D, lane);
    row_store_bf16(r, y + row * D, D, lane);
  }
}

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_bwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* dy, __nv_bfloat16* dx,
                     long long rows, int D, int accumulate) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> y, g;
    row_load_bf16(y, x + row * D, D, lane);
    const float rstd = row_layernorm_rstd(y, D, lane);
    row_load_bf16(g, dy + row * D, D, lane);
    row_layernorm_bwd(y, g, rstd, D, lane);
    if (accumulate) {
      Row<NC> o;
      row_load_bf16(o, dx + row * D, D, lane);
#pragma unroll
      for (int j = 0; j < NC; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) g.v[j][i] += o.v[j][i];
    }
    row_store_bf16(g, dx + row * D, D, lane);
  }
}

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embed_ln_fwd_kernel(const long long* tokens, const __nv_bfloat16* emb, __nv_bfloat16* cur,
                    long long rows, int D, int vocab) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    long long tok = tokens[row];
    BDH_BOUNDS_CHECK(tok, vocab, BOUNDS_EMBED_TOKEN, row);
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    Row<NC> r;
    row_load_bf16(r, emb + tok * D, D, lane);
    row_layernorm(r, D, lane);
    row_store_bf16(r, cur + row * D, D, lane);
  }
}

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embed_ln_bwd_kernel(const long long* tokens, const __nv_bfloat16* emb, const float* dcur,
                    float* demb, long long rows, int D, int vocab) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    long long tok = tokens[row];
    BDH_BOUNDS_CHECK(tok, vocab, BOUNDS_EMBED_BWD_TOKEN, row);
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    Row<NC> y, g;
    row_load_bf16(y, emb + tok * D, D, lane);
    const float rstd = row_layernorm_rstd(y, D, lane);
    row_load_f32(g, dcur + row * D, D, lane);
    row_layernorm_bwd(y, g, rstd, D, lane);
    float* dst = demb + tok * D;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      int c = (j * 32 + lane) * 8;
      if (c < D) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dst + c + i, g.v[j][i]);
      }
    }
  }
}

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
block_out_fwd_kernel(const __nv_bfloat16* cur, const __nv_bfloat16* mlp, __nv_bfloat16* out,
                     long long rows, int D) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> u, c;
    row_load_bf16(u, mlp + row * D, D, lane);
    row_layernorm(u, D, lane);
    row_load_bf16(c, cur + row * D, D, lane);
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) u.v[j][i] += c.v[j][i];
    row_layernorm(u, D, lane);
    row_store_bf16(u, out + row * D, D, lane);
  }
}

// Decode step, attention output: y = LN(a) for fp32 rows that the state-update kernel accumulated with
// atomics, and the rows are cleared for the next layer's accumulation in the same pass (one launch instead of
// a cast, a LayerNorm and a fill).
template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layernorm_f32_clear_kernel(float* a, __nv_bfloat16* y, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> u, z;
    row_load_f32(u, a + row * D, D, lane);
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) z.v[j][i] = 0.f;
    row_store_f32(z, a + row * D, D, lane, false);
    row_layernorm(u, D, lane);
    row_store_bf16(u, y + row * D, D, lane);
  }
}

// Decode step, layer tail: mlp = sum of the decoder GEMM's `parts` split-K partial tiles (fp32, part p of row r
// at part[(p * rows + r) * D]), then out = LN(cur + LN(mlp)) (one launch instead of a sum, a cast and the tail).
template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
block_out_parts_kernel(const __nv_bfloat16* cur, const float* part, int parts, __nv_bfloat16* out,
                       long long rows, int D) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> u, c;
    row_load_f32(u, part + row * D, D, lane);
    for (int p = 1; p < parts; ++p) {
      row_load_f32(c, part + (static_cast<long long>(p) * rows + row) * D, D, lane);
#pragma unroll
      for (int j = 0; j < NC; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) u.v[j][i] += c.v[j][i];
    }
    row_layernorm(u, D, lane);
    row_load_bf16(c, cur + row * D, D, lane);
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) u.v[j][i] += c.v[j][i];
    row_layernorm(u, D, lane);
    row_store_bf16(u, out + row * D, D, lane);
  }
}

template <int NC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
block_out_bwd_kernel(const __nv_bfloat16* cur, const __nv_bfloat16* mlp, const float* dout,
                     float* dcur, __nv_bfloat16* dmlp, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    Row<NC> lm, u, g;
    row_load_bf16(lm, mlp + row * D, D, lane);
    const float rstd_m = row_layernorm_rstd(lm, D, lane);  // lm = LN(mlp)
    row_load_bf16(u, cur + row * D, D, lane);
#pragma unroll
    for (int j = 0; j < NC; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) u.v[j][i] += lm.v[j][i];
    const float rstd_u = row_layernorm_rstd(u, D, lane);   // u = LN(cur + LN(mlp))
    row_load_f32(g, dout + row * D, D, lane);
    row_layernorm_bwd(u, g, rstd_u, D, lane);              // g = d(cur + LN(mlp))
    row_store_f32(g, dcur + row * D, D, lane, false);
    row_layernorm_bwd(lm, g, rstd_m, D, lane);             // g = d mlp
    row_store_bf16(g, dmlp + row * D, D, lane);
  }
}

// One warp per row of fp32 logits, V <= 1024.
__global__ void __launch_bounds__(ROW_WARPS * 32)
cross_entropy_kernel(const float* logits, const long long* targets, float* row_loss,
                     __nv_bfloat16* dlogits, long long rows, int V, float grad_scale) {
  const int lane = threadIdx.x & 31;
  long long row = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5);
  const long long stride = static_cast<long long>(gridDim.x) * ROW_WARPS;
  for (; row < rows; row += stride) {
    const float* p = logits + row * V;
    float v[32];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      int c = j * 32 + lane;
      v[j] = (c < V) ? p[c] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      int c = j * 32 + lane;
      if (c < V) {
        v[j] = __expf(v[j] - mx);
        s += v[j];
      }
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
    long long tgt = targets[row];
    if (tgt != -100) BDH_BOUNDS_CHECK(tgt, V, BOUNDS_CE_TARGET, row);
    const bool ignore = tgt < 0 || tgt >= V;
    if (lane == 0) row_loss[row] = ignore ? 0.f : (logf(s) + mx - p[tgt]);
    if (dlogits) {
      __nv_bfloat16* d = dlogits + row * V;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        int c = j * 32 + lane;
        if (c < V) {
          float gr = ignore ? 0.f : (v[j] * inv - (c == tgt ? 1.f : 0.f)) * grad_scale;
          d[c] = __float2bfloat16_rn(gr);
        }
      }
    }
  }
}

__global__ void adamw_kernel(float* __restrict__ master, const float* __restrict__ grad,
                             float* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ p16, long long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float gscale) {
  long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 w = *reinterpret_cast<float4*>(master + i);
      float4 g = *reinterpret_cast<const float4*>(grad + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* wp = &w.x; float* gp = &g.x; float* mp = &mm.x; float* vp = &vv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float gk = gp[k] * gscale;
        mp[k] = b1 * mp[k] + (1.f - b1) * gk;
        vp[k] = b2 * vp[k] + (1.f - b2) * gk * gk;
        float upd = (mp[k] / bc1) / (sqrtf(vp[k] / bc2) + eps);
        wp[k] = wp[k] * (1.f - lr * wd) - lr * upd;
      }
      *reinterpret_cast<float4*>(master + i) = w;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (p16) {
        uint2 u;
        u.x = pack_bf16x2(w.x, w.y);
        u.y = pack_bf16x2(w.z, w.w);
        *reinterpret_cast<uint2*>(p16 + i) = u;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float gk = grad[k] * gscale;
        float mk = b1 * m[k] + (1.f - b1) * gk;
        float vk = b2 * v[k] + (1.f - b2) * gk * gk;
        m[k] = mk; v[k] = vk;
        float wk = master[k] * (1.f - lr * wd) - lr * (mk / bc1) / (sqrtf(vk / bc2) + eps);
        master[k] = wk;
        if (p16) p16[k] = __float2bfloat16_rn(wk);
      }
    }
  }
}

__global__ void cast_f32_bf16_kernel(const float* in, __nv_bfloat16* out, long long n) {
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void add_f32_kernel(const float* in, float* inout, long long n) {
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) inout[i] += in[i];
}

static int row_grid(long long rows) {
  long long b = (rows + ROW_WARPS - 1) / ROW_WARPS;
  const long long cap = 148 * 16;
  return static_cast<int>(b < cap ? (b < 1 ? 1 : b) : cap);
}
static int flat_grid(long long n, int per_block) {
  long long b = (n + per_block - 1) / per_block;
  const long long cap = 148 * 8;
  return static_cast<int>(b < cap ? (b < 1 ? 1 : b) : cap);
}
static bool row_ok(int D) { return D > 0 && D <= ROW_MAX_CHUNKS * 256 && (D % 8) == 0; }
static int launch_rc() { return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH; }

#define ROW_DISPATCH(D, KERNEL, ...)                                                   \
  do {                                                                                 \
    if ((D) <= 256) KERNEL<1><<<row_grid(rows), ROW_WARPS * 32, 0, s>>>(__VA_ARGS__);       \
    else if ((D) <= 512) KERNEL<2><<<row_grid(rows), ROW_WARPS * 32, 0, s>>>(__VA_ARGS__);  \
    else if ((D) <= 1024) KERNEL<4><<<row_grid(rows), ROW_WARPS * 32, 0, s>>>(__VA_ARGS__); \
    else KERNEL<8><<<row_grid(rows), ROW_WARPS * 32, 0, s>>>(__VA_ARGS__);                  \
  } while (0)

}  // namespace bdh

using namespace bdh;
typedef __nv_bfloat16 bf16;

extern "C" int bdh_layernorm_fwd(const void* x, void* y, long long rows, int D, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, layernorm_fwd_kernel, (const bf16*)x, (bf16*)y, rows, D);
  return launch_rc();
}
extern "C" int bdh_layernorm_bwd(const void* x, const void* dy, void* dx, long long rows, int D,
                                 int accumulate, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, layernorm_bwd_kernel, (const bf16*)x, (const bf16*)dy, (bf16*)dx, rows, D, accumulate);
  return launch_rc();
}
extern "C" int bdh_embed_ln_fwd(const long long* tokens, const void* emb, void* cur, long long rows,
                                int D, int vocab, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, embed_ln_fwd_kernel, tokens, (const bf16*)emb, (bf16*)cur, rows, D, vocab);
  return launch_rc();
}
extern "C" int bdh_embed_ln_bwd(const long long* tokens, const void* emb, const float* dcur,
                                float* demb, long long rows, int D, int vocab, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, embed_ln_bwd_kernel, tokens, (const bf16*)emb, dcur, demb, rows, D, vocab);
  return launch_rc();
}
extern "C" int bdh_block_out_fwd(const void* cur, const void* mlp, void* out, long long rows, int D,
                                 cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, block_out_fwd_kernel, (const bf16*)cur, (const bf16*)mlp, (bf16*)out, rows, D);
  return launch_rc();
}
extern "C" int bdh_layernorm_f32_clear(float* a, void* y, long long rows, int D, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, layernorm_f32_clear_kernel, a, (bf16*)y, rows, D);
  return launch_rc();
}
extern "C" int bdh_block_out_parts(const void* cur, const float* part, int parts, void* out, long long rows, int D,
                                   cudaStream_t s) {
  if (!row_ok(D) || parts < 1) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, block_out_parts_kernel, (const bf16*)cur, part, parts, (bf16*)out, rows, D);
  return launch_rc();
}
extern "C" int bdh_block_out_bwd(const void* cur, const void* mlp, const float* dout, float* dcur,
                                 void* dmlp, long long rows, int D, cudaStream_t s) {
  if (!row_ok(D)) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  ROW_DISPATCH(D, block_out_bwd_kernel, (const bf16*)cur, (const bf16*)mlp, dout, dcur, (bf16*)dmlp, rows, D);
  return launch_rc();
}
extern "C" int bdh_cross_entropy(const float* logits, const long long* targets, float* row_loss,
                                 void* dlogits, long long rows, int V, float grad_scale,
                                 cudaStream_t s) {
  if (V <= 0 || V > 1024) return BDH_ERR_ARGUMENT;
  if (rows == 0) return BDH_OK;
  cross_entropy_kernel<<<row_grid(rows), ROW_WARPS * 32, 0, s>>>(logits, targets, row_loss,
                                                                 (bf16*)dlogits, rows, V, grad_scale);
  return launch_rc();
}
extern "C" int bdh_adamw(float* master, const float* grad, float* m, float* v, void* p16,
                         long long n, float lr, float beta1, float beta2, float eps, float wd,
                         int step, float grad_scale, cudaStream_t s) {
  if (n == 0) return BDH_OK;
  if (step < 1) return BDH_ERR_ARGUMENT;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  adamw_kernel<<<flat_grid(n, 1024), 256, 0, s>>>(master, grad, m, v, (bf16*)p16, n, lr, beta1, beta2,
                                                  eps, wd, bc1, bc2, grad_scale);
  return launch_rc();
}
extern "C" int bdh_cast_f32_to_bf16(const float* in, void* out, long long n, cudaStream_t s) {
  if (n == 0) return BDH_OK;
  cast_f32_bf16_kernel<<<flat_grid(n, 256), 256, 0, s>>>(in, (bf16*)out, n);
  return launch_rc();
}
extern "C" int bdh_add_f32_to_f32(const float* in, float* inout, long long n, cudaStream_t s) {
  if (n == 0) return BDH_OK;
  add_f32_kernel<<<flat_grid(n, 256), 256, 0, s>>>(in, inout, n);
  return launch_rc();
}

// ---- PoPE backward ---------------------------------------------------------------------------------
// q = softplus(x) * (cos(ph), sin(ph))  (reference: src/model/attention.rs:323-330), so
//   dx = (dq_re * cos + dq_im * sin) * sigmoid(x) + gate gradient, zero where the ReLU of x is closed.
// dq: bf16 [M, H*2N] with per-head layout [real N | imag N]; x, dxg, dx: bf16 [M, H*N]; the gate
// gradient carries the closed-gate marker (bf16 -0.0). One thread handles 8 consecutive neurons.
namespace bdh {
__global__ void pope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ x,
                                const __nv_bfloat16* __restrict__ dxg, const float* __restrict__ freqs,
                                __nv_bfloat16* __restrict__ dx, long long M, int H, int N, int T, int pos0) {
  const long long per_row = static_cast<long long>(H) * N / 8;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = M * per_row, stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (; i < total; i += stride) {
    const long long m = i / per_row;
    const int c = static_cast<int>(i % per_row) * 8;     // column in [0, H*N)
    const int h = c / N, n = c % N;
    const float pos = static_cast<float>(pos0 + static_cast<int>(m % T));
    const long long off = m * H * N + c;
    const long long qoff = m * 2 * H * N + static_cast<long long>(h) * 2 * N + n;
    uint4 ux = *reinterpret_cast<const uint4*>(x + off);
    uint4 ug = *reinterpret_cast<const uint4*>(dxg + off);
    uint4 ur = *reinterpret_cast<const uint4*>(dq + qoff);
    uint4 ui = *reinterpret_cast<const uint4*>(dq + qoff + N);
    const uint32_t* px = &ux.x; const uint32_t* pg = &ug.x; const uint32_t* pr = &ur.x; const uint32_t* pi = &ui.x;
    uint4 out;
    uint32_t* po = &out.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 xv = unpack_bf16x2(px[k]), gv = unpack_bf16x2(pg[k]), rv = unpack_bf16x2(pr[k]), iv = unpack_bf16x2(pi[k]);
      float res[2];
      const float xs[2] = {xv.x, xv.y}, gs[2] = {gv.x, gv.y}, rs[2] = {rv.x, rv.y}, is[2] = {iv.x, iv.y};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float raw = pos * __ldg(freqs + n + 2 * k + j);
        float ph = (raw - floorf(raw)) * 6.283185307179586f;
        float s, co;
        __sincosf(ph, &s, &co);
        const float sig = 1.f / (1.f + __expf(-xs[j]));
        res[j] = (xs[j] > 0.f) ? (rs[j] * co + is[j] * s) * sig + gs[j] : 0.f;
      }
      po[k] = pack_bf16x2(res[0], res[1]);
    }
    *reinterpret_cast<uint4*>(dx + off) = out;
  }
}
}  // namespace bdh

extern "C" int bdh_pope_bwd(const void* dq, const void* x, const void* dxg, const float* freqs, void* dx, long long M,
                            int H, int N, int T, int pos0, cudaStream_t s) {
  if (M <= 0 || H <= 0 || N <= 0 || (N % 8) || T <= 0) return BDH_ERR_ARGUMENT;
  const long long total = M * H * N / 8;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  bdh::pope_bwd_kernel<<<static_cast<int>(blocks), 256, 0, s>>>((const bf16*)dq, (const bf16*)x, (const bf16*)dxg, freqs,
                                                               (bf16*)dx, M, H, N, T, pos0);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// ---- PoPE query from the stored x -------------------------------------------------------------------
// q = softplus(x) * (cos(ph), sin(ph)) written again from the bf16 x that the encoder stored, so that the
// backward pass need not keep q (twice the width of x) for every layer: x bf16 [M, H*N] -> q bf16 [M, H*2N]
// with the per-head layout [real N | imag N]. One thread handles 8 consecutive neurons.
namespace bdh {
__global__ void pope_rotate_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ freqs,
                                   __nv_bfloat16* __restrict__ q, long long M, int H, int N, int T, int pos0) {
  const long long per_row = static_cast<long long>(H) * N / 8;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = M * per_row, stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (; i < total; i += stride) {
    const long long m = i / per_row;
    const int c = static_cast<int>(i % per_row) * 8;
    const int h = c / N, n = c % N;
    const float pos = static_cast<float>(pos0 + static_cast<int>(m % T));
    const long long qoff = m * 2 * H * N + static_cast<long long>(h) * 2 * N + n;
    const uint4 ux = *reinterpret_cast<const uint4*>(x + m * H * N + c);
    const uint32_t* px = &ux.x;
    uint4 re, im;
    uint32_t* pr = &re.x;
    uint32_t* pi = &im.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 xv = unpack_bf16x2(px[k]);
      const float xs[2] = {xv.x, xv.y};
      float r[2], g[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float raw = pos * __ldg(freqs + n + 2 * k + j);
        const float ph = (raw - floorf(raw)) * 6.283185307179586f;
        float s, co;
        __sincosf(ph, &s, &co);
        const float mag = xs[j] + __logf(1.f + __expf(-xs[j]));      // softplus of a non-negative value
        r[j] = mag * co;
        g[j] = mag * s;
      }
      pr[k] = pack_bf16x2(r[0], r[1]);
      pi[k] = pack_bf16x2(g[0], g[1]);
    }
    *reinterpret_cast<uint4*>(q + qoff) = re;
    *reinterpret_cast<uint4*>(q + qoff + N) = im;
  }
}
}  // namespace bdh

extern "C" int bdh_pope_rotate(const void* x, const float* freqs, void* q, long long M, int H, int N, int T, int pos0,
                               cudaStream_t s) {
  if (M <= 0 || H <= 0 || N <= 0 || (N % 8) || T <= 0) return BDH_ERR_ARGUMENT;
  const long long total = M * H * N / 8;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  bdh::pope_rotate_kernel<<<static_cast<int>(blocks), 256, 0, s>>>((const bf16*)x, freqs, (bf16*)q, M, H, N, T, pos0);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// ---- state scans of the chunk-state attention -------------------------------------------------------------
// The [N', D] states of the J segments of a sequence are independent per element, so the hand-off is an
// elementwise recurrence over j. seg / d_rin: fp32 [B, J, H, per] (per = N' * D); start / init / total: fp32
// [B, H, per]; decay: g^C per head (nullptr: 1). One thread owns four consecutive elements of one (b, h).
//   forward : run = start; for j = 0..J-1: out16[j] = run; run = run * g + seg[j];          total = run
//   backward: acc = init;  for j = J-1..0: out16[j] = acc; acc = d_rin[j] + acc * g  (the last update is unused)
// out16 is bf16: the state every segment starts from (forward), the gradient of every segment's own state
// (backward) - both are GEMM operands next.
namespace bdh {
template <bool BWD>
__global__ void __launch_bounds__(256)
state_scan_kernel(const float* __restrict__ seg, const float* __restrict__ start, const float* __restrict__ decay,
                  __nv_bfloat16* __restrict__ out16, float* __restrict__ total, long long per4, int J, int H,
                  long long n_bh) {
  const long long n = n_bh * per4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long bh = i / per4, e = i - bh * per4;
    const long long b = bh / H;
    const int h = static_cast<int>(bh - b * H);
    const float g = decay ? __ldg(decay + h) : 1.f;
    float4 run = start ? reinterpret_cast<const float4*>(start)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int jj = 0; jj < J; ++jj) {
      const int j = BWD ? J - 1 - jj : jj;
      const long long at = ((b * J + j) * H + h) * per4 + e;
      uint2 u;
      u.x = pack_bf16x2(run.x, run.y);
      u.y = pack_bf16x2(run.z, run.w);
      reinterpret_cast<uint2*>(out16)[at] = u;
      if (BWD && j == 0) break;
      const float4 s = __ldcs(reinterpret_cast<const float4*>(seg) + at);
      run.x = run.x * g + s.x; run.y = run.y * g + s.y; run.z = run.z * g + s.z; run.w = run.w * g + s.w;
    }
    if (!BWD && total) reinterpret_cast<float4*>(total)[i] = run;
  }
}
}  // namespace bdh

extern "C" int bdh_state_scan(const float* seg, const float* start, const float* decay, void* out16, float* total,
                              long long per, int J, int H, long long n_bh, int backward, cudaStream_t s) {
  if (per <= 0 || (per % 4) || J < 1 || H < 1 || n_bh < 1) return BDH_ERR_ARGUMENT;
  const long long n = n_bh * (per / 4);
  long long blocks = (n + 255) / 256;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (backward)
    bdh::state_scan_kernel<true><<<static_cast<int>(blocks), 256, 0, s>>>(seg, start, decay, (bf16*)out16, total, per / 4, J, H, n_bh);
  else
    bdh::state_scan_kernel<false><<<static_cast<int>(blocks), 256, 0, s>>>(seg, start, decay, (bf16*)out16, total, per / 4, J, H, n_bh);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// ---- L1 row normalisation of strictly causal scores (the `forward_fast` attention) -------------
// S is bf16 [rows, T] with rows = (batch, head, t); only columns s < t of row t carry scores
// (reference: src/model/attention.rs:142-175: tril(-1), then S / (sum_j |S_ij| + 1e-6)).
//   forward : S <- S / r,  r = sum_{s<t} |S| + 1e-6           (r is kept for the backward pass)
//   backward: G <- (G - sign(Sn) * sum_{s<t} G Sn) / r         (Sn = normalised scores)
// One warp per row, 8 columns per lane per step; columns s >= t are left untouched.
namespace bdh {
template <bool BWD>
__global__ void __launch_bounds__(256)
rownorm_kernel(__nv_bfloat16* __restrict__ S, const __nv_bfloat16* __restrict__ Sn, float* __restrict__ rnorm,
               long long rows, int T, int ld) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int t = static_cast<int>(row % T);
  __nv_bfloat16* p = S + row * ld;
  const __nv_bfloat16* pn = BWD ? Sn + row * ld : nullptr;
  float acc = 0.f;
  for (int s0 = lane * 8; s0 < t; s0 += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(p + s0);
    const uint32_t* w = &u.x;
    uint4 un = make_uint4(0, 0, 0, 0);
    if (BWD) un = *reinterpret_cast<const uint4*>(pn + s0);
    const uint32_t* wn = &un.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16x2(w[k]);
      const bool in0 = s0 + 2 * k < t, in1 = s0 + 2 * k + 1 < t;
      if (BWD) {
        const float2 b = unpack_bf16x2(wn[k]);
        acc += (in0 ? a.x * b.x : 0.f) + (in1 ? a.y * b.y : 0.f);
      } else {
        acc += (in0 ? fabsf(a.x) : 0.f) + (in1 ? fabsf(a.y) : 0.f);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  float r;
  if (BWD) {
    r = rnorm[row];
  } else {
    r = acc + 1e-6f;
    if (lane == 0) rnorm[row] = r;
  }
  const float inv = 1.f / r;
  for (int s0 = lane * 8; s0 < t; s0 += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(p + s0);
    uint32_t* w = &u.x;
    uint4 un = make_uint4(0, 0, 0, 0);
    if (BWD) un = *reinterpret_cast<const uint4*>(pn + s0);
    const uint32_t* wn = &un.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16x2(w[k]);
      const bool in0 = s0 + 2 * k < t, in1 = s0 + 2 * k + 1 < t;
      if (BWD) {
        const float2 b = unpack_bf16x2(wn[k]);
        const float s0v = (b.x > 0.f) ? 1.f : (b.x < 0.f ? -1.f : 0.f);
        const float s1v = (b.y > 0.f) ? 1.f : (b.y < 0.f ? -1.f : 0.f);
        a.x = in0 ? (a.x - s0v * acc) * inv : a.x;
        a.y = in1 ? (a.y - s1v * acc) * inv : a.y;
      } else {
        a.x = in0 ? a.x * inv : a.x;
        a.y = in1 ? a.y * inv : a.y;
      }
      w[k] = pack_bf16x2(a.x, a.y);
    }
    *reinterpret_cast<uint4*>(p + s0) = u;
  }
}
}  // namespace bdh

extern "C" int bdh_rownorm_fwd(void* scores_bf16, float* rnorm, long long rows, int T, int ld, cudaStream_t s) {
  if (rows <= 0 || T <= 0 || (ld % 8) || ld < T) return BDH_ERR_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(scores_bf16) & 15) return BDH_ERR_ALIGNMENT;
  const long long blocks = (rows + 7) / 8;
  bdh::rownorm_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, s>>>((bf16*)scores_bf16, nullptr, rnorm, rows, T, ld);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

extern "C" int bdh_rownorm_bwd(void* grad_bf16, const void* normed_bf16, const float* rnorm, long long rows, int T,
                               int ld, cudaStream_t s) {
  if (rows <= 0 || T <= 0 || (ld % 8) || ld < T) return BDH_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(grad_bf16) | reinterpret_cast<uintptr_t>(normed_bf16)) & 15) return BDH_ERR_ALIGNMENT;
  const long long blocks = (rows + 7) / 8;
  bdh::rownorm_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, s>>>((bf16*)grad_bf16, (const bf16*)normed_bf16,
                                                                        const_cast<float*>(rnorm), rows, T, ld);
  return cudaGetLastError() == cudaSuccess ? BDH_OK : BDH_ERR_LAUNCH;
}

// First data-dependent index of this file's kernels that was out of range since the last clear:
// out = {checked build?, site, index, extent, where} (csrc/debug_bounds.cuh).
extern "C" int bdh_bounds_record_rowwise(long long* out5, int clear) { return bdh::bounds_record_read(out5, clear) ? BDH_ERR_LAUNCH : BDH_OK; }
