// torch.ops.bdh.* : thin argument-checking shims from torch tensors to the C kernel interface.
// All outputs are allocated by the Python caller; nothing here allocates device memory except
// the one-word status buffer created on first use.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <vector>

#include "bdh_kernels.h"

namespace {

using at::Tensor;
using c10::optional;

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == BDH_OK, "bdh kernel '", what, "' failed with code ", rc);
}

Tensor& status_word() {
  static Tensor t;
  if (!t.defined()) t = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA));
  return t;
}

BdhMat as_mat(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1,
              name, ": expected a 2-D bf16 CUDA tensor with unit column stride");
  return BdhMat{t.data_ptr(), t.size(0), t.size(1), t.stride(0)};
}

const void* opt_ptr(const optional<Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
long long opt_ld(const optional<Tensor>& t) {
  return (t.has_value() && t->dim() >= 2) ? t->stride(t->dim() - 2) : 0;
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void gemm(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, int64_t M, int64_t N, int64_t K,
          int64_t nz0, int64_t nz1, at::IntArrayRef a_off, at::IntArrayRef b_off, int64_t epi,
          int64_t flags, const optional<Tensor>& out0, const optional<Tensor>& out1,
          const optional<Tensor>& in0, const optional<Tensor>& in1, at::IntArrayRef c_off,
          at::IntArrayRef o1_off, double alpha, double theta, int64_t T, int64_t pos0,
          int64_t n_per_head, const optional<Tensor>& freqs, const optional<Tensor>& slopes,
          int64_t causal_tiles, int64_t causal_k, int64_t bn, int64_t max_ctas, bool tma_epilogue, int64_t mc_out, double drop_p, int64_t drop_seed,
          at::IntArrayRef peer_ptrs, int64_t peer_rows, int64_t peer_rank, const optional<Tensor>& bias,
          at::IntArrayRef gather_ptrs, int64_t gather_rows, int64_t gather_rank, const optional<Tensor>& gather_arrived,
          const optional<Tensor>& tile_skip) {
  c10::cuda::CUDAGuard guard(a.device());
  BdhMat A = as_mat(a, "a"), B = as_mat(b, "b");
  TORCH_CHECK(a_off.size() == 4 && b_off.size() == 4 && c_off.size() == 4 && o1_off.size() == 3,
              "offset lists must have 4/4/4/3 entries");
  BdhGemmDesc d{};
  d.M = M; d.N = N; d.K = K; d.nz0 = nz0; d.nz1 = nz1;
  for (int i = 0; i < 4; ++i) { d.a_off[i] = a_off[i]; d.b_off[i] = b_off[i]; d.c_off[i] = c_off[i]; }
  for (int i = 0; i < 3; ++i) d.o1_off[i] = o1_off[i];
  d.epi = epi; d.flags = flags; d.bn = bn;
  d.causal_tiles = causal_tiles; d.causal_k = causal_k;
  d.out0 = const_cast<void*>(opt_ptr(out0)); d.out1 = const_cast<void*>(opt_ptr(out1));
  d.in0 = opt_ptr(in0); d.in1 = opt_ptr(in1);
  d.ld_out0 = opt_ld(out0); d.ld_out1 = opt_ld(out1); d.ld_in0 = opt_ld(in0); d.ld_in1 = opt_ld(in1);
  d.alpha = alpha; d.theta = theta; d.T = T; d.pos0 = pos0; d.n_per_head = n_per_head;
  d.freqs = freqs.has_value() ? freqs->data_ptr<float>() : nullptr;
  d.slopes = slopes.has_value() ? slopes->data_ptr<float>() : nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->scalar_type() == at::kFloat, "bias: contiguous fp32");
    d.bias = bias->data_ptr<float>();
  }
  d.status = status_word().data_ptr<int>();
  d.max_ctas = max_ctas;
  d.no_tma_epilogue = tma_epilogue ? 0 : 1;
  d.drop_p = drop_p; d.drop_seed = static_cast<unsigned>(drop_seed);
  if (mc_out != 0) d.out0 = reinterpret_cast<void*>(mc_out);   // multicast mapping of out0 (EPI_F_MC_RED)
  long long peers[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (!peer_ptrs.empty()) {                                      // reduce-scatter epilogue (EPI_F_PEER_RS)
    TORCH_CHECK(peer_ptrs.size() <= 8, "at most 8 peers");
    for (size_t i = 0; i < peer_ptrs.size(); ++i) peers[i] = peer_ptrs[i];
    d.peer_out = peers; d.peer_world = static_cast<int>(peer_ptrs.size()); d.peer_rows = peer_rows; d.peer_rank = static_cast<int>(peer_rank);
  }
  long long gsrc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (gather_ptrs.size() > 1) {                                  // all-gather of A inside the kernel
    TORCH_CHECK(gather_ptrs.size() <= 8, "at most 8 peers");
    TORCH_CHECK(gather_arrived.has_value() && gather_arrived->is_cuda() && gather_arrived->is_contiguous() &&
                gather_arrived->scalar_type() == at::kInt && gather_arrived->numel() >= (M + 127) / 128,
                "gather_arrived: int32 counters, one per 128 rows of A");
    for (size_t i = 0; i < gather_ptrs.size(); ++i) gsrc[i] = gather_ptrs[i];
    d.gather_src = gsrc; d.gather_world = static_cast<int>(gather_ptrs.size()); d.gather_rows = gather_rows;
    d.gather_rank = static_cast<int>(gather_rank);
    d.gather_arrived = reinterpret_cast<unsigned*>(gather_arrived->data_ptr<int>());
  }
  if (tile_skip.has_value()) {
    const int64_t bn_ = bn == 128 ? 128 : 256;
    TORCH_CHECK(tile_skip->is_cuda() && tile_skip->is_contiguous() && tile_skip->scalar_type() == at::kByte &&
                tile_skip->numel() == ((M + 127) / 128) * ((N + bn_ - 1) / bn_) && epi == 3,
                "tile_skip: uint8 [ceil(M/128), ceil(N/bn)], causal epilogue only");
    d.tile_skip = tile_skip->data_ptr<unsigned char>();
  }
  check_rc(bdh_gemm_bf16(&A, a_mn, &B, b_mn, &d, cur_stream()), "gemm_bf16");
}

BdhDualDesc dual_desc(int64_t M, int64_t H, int64_t n_per_head, int64_t K1, int64_t N2, int64_t T, int64_t group_per_head,
                      int64_t max_ctas, Tensor& partials) {
  TORCH_CHECK(partials.is_cuda() && partials.is_contiguous() && partials.scalar_type() == at::kFloat,
              "partials: expected a contiguous fp32 CUDA tensor");
  BdhDualDesc d{};
  d.M = M; d.H = H; d.n_per_head = n_per_head; d.K1 = K1; d.N2 = N2; d.T = T;
  d.group_per_head = group_per_head;
  d.max_ctas = max_ctas;
  d.partials = partials.data_ptr<float>();
  d.partial_floats = partials.numel();
  d.status = status_word().data_ptr<int>();
  return d;
}

int64_t dual_gemm_partial_floats(int64_t M, int64_t H, int64_t n_per_head, int64_t N2, int64_t group_per_head,
                                 int64_t max_ctas) {
  BdhDualDesc d{};
  d.M = M; d.H = H; d.n_per_head = n_per_head; d.N2 = N2; d.group_per_head = group_per_head; d.max_ctas = max_ctas;
  return bdh_dual_gemm_partial_floats(&d);
}

void dual_gemm(const Tensor& a1, const Tensor& b1, bool b1_mn, const Tensor& b2, Tensor& p, int64_t M, int64_t H,
               int64_t n_per_head, int64_t K1, int64_t N2, int64_t T, int64_t epi, int64_t flags, int64_t group_per_head,
               int64_t a1_b, int64_t a1_h, int64_t b1_b, const optional<Tensor>& in0, const optional<Tensor>& in1,
               const optional<Tensor>& out1, double alpha, double theta, int64_t pos0, double drop_p, int64_t drop_seed,
               Tensor& partials, int64_t max_ctas) {
  c10::cuda::CUDAGuard guard(a1.device());
  BdhMat A1 = as_mat(a1, "a1"), B1 = as_mat(b1, "b1"), B2 = as_mat(b2, "b2"), P = as_mat(p, "p");
  BdhDualDesc d = dual_desc(M, H, n_per_head, K1, N2, T, group_per_head, max_ctas, partials);
  d.epi = epi; d.flags = flags;
  d.a1_b = a1_b; d.a1_h = a1_h; d.b1_b = b1_b;
  d.in0 = opt_ptr(in0); d.in1 = opt_ptr(in1); d.out1 = const_cast<void*>(opt_ptr(out1));
  d.ld_in0 = opt_ld(in0); d.ld_in1 = opt_ld(in1); d.ld_out1 = opt_ld(out1);
  d.alpha = alpha; d.theta = theta; d.pos0 = pos0;
  d.drop_p = drop_p; d.drop_seed = static_cast<unsigned>(drop_seed);
  // every window the kernel addresses has to lie inside its tensor
  const int64_t HN = H * n_per_head;
  TORCH_CHECK(p.size(0) >= M && p.size(1) >= HN, "p: expected at least [M, H*n_per_head]");
  TORCH_CHECK(b2.size(0) >= HN && b2.size(1) >= N2, "b2: expected at least [H*n_per_head, N2]");
  for (const optional<Tensor>* t : {&in0, &out1})
    if (t->has_value()) TORCH_CHECK((*t)->dim() == 2 && (*t)->size(0) >= M && (*t)->size(1) >= HN && (*t)->stride(1) == 1);
  if (in1.has_value()) {
    const bool table = epi == 5;
    TORCH_CHECK(in1->dim() == 2 && in1->stride(1) == 1 && in1->size(0) >= (table ? T : M) &&
                in1->size(1) >= (table ? n_per_head : HN), "in1: window leaves the tensor");
  }
  check_rc(bdh_dual_gemm(&A1, &B1, b1_mn, &B2, &P, &d, cur_stream()), "dual_gemm");
}

void dual_gemm_reduce(Tensor& partials, int64_t M, int64_t H, int64_t n_per_head, int64_t N2, int64_t group_per_head,
                      int64_t max_ctas, Tensor& out, bool accumulate, int64_t out_h_stride) {
  c10::cuda::CUDAGuard guard(out.device());
  BdhDualDesc d = dual_desc(M, H, n_per_head, 64, N2, 128, group_per_head, max_ctas, partials);
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(1) >= N2);
  const bool bf = out.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || out.scalar_type() == at::kFloat, "out: bf16 or fp32");
  TORCH_CHECK(out.size(0) >= (group_per_head ? (H - 1) * out_h_stride + M : M), "out: too few rows");
  TORCH_CHECK(partials.numel() >= dual_gemm_partial_floats(M, H, n_per_head, N2, group_per_head, max_ctas));
  check_rc(bdh_dual_gemm_reduce(&d, out.data_ptr(), out.stride(0), bf ? 1 : 0, accumulate ? 1 : 0, out_h_stride,
                                cur_stream()), "dual_gemm_reduce");
}

void rownorm_fwd(Tensor& scores, Tensor& rnorm, int64_t T) {
  c10::cuda::CUDAGuard guard(scores.device());
  TORCH_CHECK(scores.is_cuda() && scores.dim() == 2 && scores.scalar_type() == at::kBFloat16 && scores.stride(1) == 1);
  TORCH_CHECK(rnorm.is_cuda() && rnorm.is_contiguous() && rnorm.scalar_type() == at::kFloat && rnorm.numel() == scores.size(0));
  check_rc(bdh_rownorm_fwd(scores.data_ptr(), rnorm.data_ptr<float>(), scores.size(0), T, scores.stride(0), cur_stream()),
           "rownorm_fwd");
}
void rownorm_bwd(Tensor& grad, const Tensor& normed, const Tensor& rnorm, int64_t T) {
  c10::cuda::CUDAGuard guard(grad.device());
  TORCH_CHECK(grad.is_cuda() && grad.dim() == 2 && grad.scalar_type() == at::kBFloat16 && grad.stride(1) == 1);
  TORCH_CHECK(normed.scalar_type() == at::kBFloat16 && normed.sizes() == grad.sizes() && normed.stride(0) == grad.stride(0));
  TORCH_CHECK(rnorm.is_contiguous() && rnorm.scalar_type() == at::kFloat && rnorm.numel() == grad.size(0));
  check_rc(bdh_rownorm_bwd(grad.data_ptr(), normed.data_ptr(), rnorm.data_ptr<float>(), grad.size(0), T, grad.stride(0),
                           cur_stream()), "rownorm_bwd");
}

void check_rows(const Tensor& t, int64_t D, at::ScalarType st, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == st && t.size(-1) == D, name,
              ": expected a contiguous CUDA tensor with last dim ", D);
}

void layernorm_fwd(const Tensor& x, Tensor& y) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t D = x.size(-1);
  check_rows(x, D, at::kBFloat16, "x"); check_rows(y, D, at::kBFloat16, "y");
  check_rc(bdh_layernorm_fwd(x.data_ptr(), y.data_ptr(), x.numel() / D, D, cur_stream()), "layernorm_fwd");
}
void layernorm_bwd(const Tensor& x, const Tensor& dy, Tensor& dx, bool accumulate) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t D = x.size(-1);
  check_rows(x, D, at::kBFloat16, "x"); check_rows(dy, D, at::kBFloat16, "dy"); check_rows(dx, D, at::kBFloat16, "dx");
  check_rc(bdh_layernorm_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.numel() / D, D, accumulate, cur_stream()),
           "layernorm_bwd");
}
void embed_ln_fwd(const Tensor& tokens, const Tensor& emb, Tensor& cur) {
  c10::cuda::CUDAGuard guard(emb.device());
  const int64_t D = emb.size(1);
  TORCH_CHECK(tokens.scalar_type() == at::kLong && tokens.is_contiguous() && tokens.is_cuda());
  check_rows(emb, D, at::kBFloat16, "emb"); check_rows(cur, D, at::kBFloat16, "cur");
  check_rc(bdh_embed_ln_fwd(tokens.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()) : nullptr,
                            emb.data_ptr(), cur.data_ptr(), tokens.numel(), D, emb.size(0), cur_stream()),
           "embed_ln_fwd");
}
void embed_ln_bwd(const Tensor& tokens, const Tensor& emb, const Tensor& dcur, Tensor& demb) {
  c10::cuda::CUDAGuard guard(emb.device());
  const int64_t D = emb.size(1);
  TORCH_CHECK(tokens.scalar_type() == at::kLong && tokens.is_contiguous() && tokens.is_cuda());
  check_rows(emb, D, at::kBFloat16, "emb"); check_rows(dcur, D, at::kFloat, "dcur"); check_rows(demb, D, at::kFloat, "demb");
  check_rc(bdh_embed_ln_bwd(reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()), emb.data_ptr(),
                            dcur.data_ptr<float>(), demb.data_ptr<float>(), tokens.numel(), D, emb.size(0), cur_stream()),
           "embed_ln_bwd");
}
void block_out_fwd(const Tensor& cur, const Tensor& mlp, Tensor& out) {
  c10::cuda::CUDAGuard guard(cur.device());
  const int64_t D = cur.size(-1);
  check_rows(cur, D, at::kBFloat16, "cur"); check_rows(mlp, D, at::kBFloat16, "mlp"); check_rows(out, D, at::kBFloat16, "out");
  check_rc(bdh_block_out_fwd(cur.data_ptr(), mlp.data_ptr(), out.data_ptr(), cur.numel() / D, D, cur_stream()), "block_out_fwd");
}
void layernorm_f32_clear(Tensor& a, Tensor& y) {
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t D = a.size(-1);
  check_rows(a, D, at::kFloat, "a"); check_rows(y, D, at::kBFloat16, "y");
  TORCH_CHECK(a.numel() == y.numel(), "layernorm_f32_clear: shapes differ");
  check_rc(bdh_layernorm_f32_clear(a.data_ptr<float>(), y.data_ptr(), a.numel() / D, D, cur_stream()), "layernorm_f32_clear");
}
void block_out_parts(const Tensor& cur, const Tensor& part, Tensor& out) {
  c10::cuda::CUDAGuard guard(cur.device());
  const int64_t D = cur.size(-1);
  check_rows(cur, D, at::kBFloat16, "cur"); check_rows(part, D, at::kFloat, "part"); check_rows(out, D, at::kBFloat16, "out");
  TORCH_CHECK(cur.numel() > 0 && part.numel() % cur.numel() == 0 && out.numel() == cur.numel(),
              "block_out_parts: part must hold a whole number of [rows, D] tiles");
  check_rc(bdh_block_out_parts(cur.data_ptr(), part.data_ptr<float>(), static_cast<int>(part.numel() / cur.numel()),
                               out.data_ptr(), cur.numel() / D, D, cur_stream()), "block_out_parts");
}
void block_out_bwd(const Tensor& cur, const Tensor& mlp, const Tensor& dout, Tensor& dcur, Tensor& dmlp) {
  c10::cuda::CUDAGuard guard(cur.device());
  const int64_t D = cur.size(-1);
  check_rows(cur, D, at::kBFloat16, "cur"); check_rows(mlp, D, at::kBFloat16, "mlp");
  check_rows(dout, D, at::kFloat, "dout"); check_rows(dcur, D, at::kFloat, "dcur"); check_rows(dmlp, D, at::kBFloat16, "dmlp");
  check_rc(bdh_block_out_bwd(cur.data_ptr(), mlp.data_ptr(), dout.data_ptr<float>(), dcur.data_ptr<float>(), dmlp.data_ptr(),
                             cur.numel() / D, D, cur_stream()), "block_out_bwd");
}
void cross_entropy(const Tensor& logits, const Tensor& targets, Tensor& row_loss, const optional<Tensor>& dlogits,
                   double grad_scale) {
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t V = logits.size(-1);
  check_rows(logits, V, at::kFloat, "logits");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.is_cuda());
  TORCH_CHECK(row_loss.scalar_type() == at::kFloat && row_loss.is_contiguous() && row_loss.numel() == targets.numel());
  if (dlogits.has_value()) check_rows(*dlogits, V, at::kBFloat16, "dlogits");
  check_rc(bdh_cross_entropy(logits.data_ptr<float>(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                             row_loss.data_ptr<float>(), const_cast<void*>(opt_ptr(dlogits)), targets.numel(), V,
                             grad_scale, cur_stream()), "cross_entropy");
}
void adamw(Tensor& master, const Tensor& grad, Tensor& m, Tensor& v, const optional<Tensor>& p16, double lr, double beta1,
           double beta2, double eps, double wd, int64_t step, double grad_scale) {
  c10::cuda::CUDAGuard guard(master.device());
  const int64_t n = master.numel();
  for (const Tensor* t : std::initializer_list<const Tensor*>{&master, &grad, &m, &v})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat && t->numel() == n);
  if (p16.has_value()) TORCH_CHECK(p16->is_contiguous() && p16->scalar_type() == at::kBFloat16 && p16->numel() == n);
  check_rc(bdh_adamw(master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                     const_cast<void*>(opt_ptr(p16)), n, lr, beta1, beta2, eps, wd, step, grad_scale, cur_stream()), "adamw");
}

Tensor status() { return status_word(); }

// int64 [2, 5] on the host: rows = the kernels of rowwise.cu, of graph.cu; columns = {checked build?,
// site, index, extent, where} of the first out-of-range data-dependent index (csrc/debug_bounds.cuh).
// Synchronises the current device.
Tensor bounds_records(bool clear) {
  Tensor out = at::zeros({2, 5}, at::TensorOptions().dtype(at::kLong));
  long long* p = reinterpret_cast<long long*>(out.data_ptr<int64_t>());
  check_rc(bdh_bounds_record_rowwise(p, clear ? 1 : 0), "bounds_record_rowwise");
  check_rc(bdh_bounds_record_graph(p + 5, clear ? 1 : 0), "bounds_record_graph");
  return out;
}

std::vector<long long> as_ptrs(at::IntArrayRef v) { return std::vector<long long>(v.begin(), v.end()); }

// `anchor` only selects the device / stream; the buffers are addressed through the pointer lists.
void allreduce_scale(const Tensor& anchor, at::IntArrayRef buf_ptrs, at::IntArrayRef flag_ptrs, int64_t mc_ptr,
                     int64_t rank, int64_t world, int64_t n_floats, double scale, int64_t epoch, int64_t ctas) {
  c10::cuda::CUDAGuard guard(anchor.device());
  TORCH_CHECK((int64_t)buf_ptrs.size() == world && (int64_t)flag_ptrs.size() == world);
  auto b = as_ptrs(buf_ptrs), f = as_ptrs(flag_ptrs);
  check_rc(bdh_allreduce_scale(b.data(), f.data(), mc_ptr, rank, world, n_floats, scale, (unsigned)epoch, ctas,
                               status_word().data_ptr<int>(), cur_stream()), "allreduce_scale");
}

void gather_blocks(const Tensor& anchor, at::IntArrayRef slot_ptrs, at::IntArrayRef flag_ptrs,
                   at::IntArrayRef out_ptrs, int64_t out_mc, bool out_bf16, int64_t rank, int64_t world,
                   int64_t block_floats, int64_t epoch, int64_t ctas) {
  c10::cuda::CUDAGuard guard(anchor.device());
  TORCH_CHECK((int64_t)slot_ptrs.size() == world && (int64_t)flag_ptrs.size() == world &&
              (int64_t)out_ptrs.size() == world);
  auto b = as_ptrs(slot_ptrs), f = as_ptrs(flag_ptrs), o = as_ptrs(out_ptrs);
  check_rc(bdh_gather_blocks(b.data(), f.data(), o.data(), out_mc, out_bf16 ? 1 : 0, rank, world, block_floats,
                             (unsigned)epoch, ctas, status_word().data_ptr<int>(), cur_stream()), "gather_blocks");
}

void rs_adamw_ag(const Tensor& anchor, at::IntArrayRef grad_ptrs, at::IntArrayRef flag_ptrs, int64_t grad_mc,
                 at::IntArrayRef shadow_ptrs, int64_t rank, int64_t world, int64_t n_floats, Tensor& master,
                 Tensor& m, Tensor& v, double lr, double beta1, double beta2, double eps, double wd, int64_t step,
                 double grad_scale, int64_t epoch, int64_t ctas) {
  c10::cuda::CUDAGuard guard(anchor.device());
  TORCH_CHECK((int64_t)grad_ptrs.size() == world && (int64_t)flag_ptrs.size() == world &&
              (int64_t)shadow_ptrs.size() == world);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&master, &m, &v})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat);
  auto g = as_ptrs(grad_ptrs), f = as_ptrs(flag_ptrs), sh = as_ptrs(shadow_ptrs);
  check_rc(bdh_rs_adamw_ag(g.data(), f.data(), grad_mc, sh.data(), rank, world, n_floats, master.data_ptr<float>(),
                           m.data_ptr<float>(), v.data_ptr<float>(), lr, beta1, beta2, eps, wd, step, grad_scale,
                           (unsigned)epoch, ctas, status_word().data_ptr<int>(), cur_stream()), "rs_adamw_ag");
}

void shard_adamw_ag(at::IntArrayRef flag_ptrs, at::IntArrayRef shadow_ptrs, int64_t rank, int64_t world, Tensor& gacc,
                    Tensor& master, Tensor& m, Tensor& v, at::IntArrayRef seg_lo, at::IntArrayRef seg_dst, double lr,
                    double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale, int64_t epoch,
                    int64_t ctas) {
  c10::cuda::CUDAGuard guard(master.device());
  TORCH_CHECK((int64_t)flag_ptrs.size() == world && (int64_t)shadow_ptrs.size() == world);
  TORCH_CHECK(seg_lo.size() == seg_dst.size() + 1 && !seg_dst.empty() && seg_dst.size() <= 4);
  for (const Tensor* t : std::initializer_list<const Tensor*>{&gacc, &master, &m, &v})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat && t->numel() >= seg_lo.back());
  auto f = as_ptrs(flag_ptrs), sh = as_ptrs(shadow_ptrs);
  std::vector<long long> lo(seg_lo.begin(), seg_lo.end()), dst(seg_dst.begin(), seg_dst.end());
  check_rc(bdh_shard_adamw_ag(f.data(), sh.data(), rank, world, gacc.data_ptr<float>(), master.data_ptr<float>(),
                              m.data_ptr<float>(), v.data_ptr<float>(), (int)dst.size(), lo.data(), dst.data(), lr, beta1,
                              beta2, eps, wd, step, grad_scale, (unsigned)epoch, ctas, status_word().data_ptr<int>(),
                              cur_stream()), "shard_adamw_ag");
}

void shard_bcast(at::IntArrayRef flag_ptrs, at::IntArrayRef out_ptrs, int64_t out_mc, int64_t rank, int64_t world, Tensor& gacc,
                 at::IntArrayRef seg_lo, at::IntArrayRef seg_dst, double scale, int64_t epoch, int64_t ctas) {
  c10::cuda::CUDAGuard guard(gacc.device());
  TORCH_CHECK((int64_t)flag_ptrs.size() == world && (int64_t)out_ptrs.size() == world);
  TORCH_CHECK(seg_lo.size() == seg_dst.size() + 1 && !seg_dst.empty() && seg_dst.size() <= 4);
  TORCH_CHECK(gacc.is_cuda() && gacc.is_contiguous() && gacc.scalar_type() == at::kFloat && gacc.numel() >= seg_lo.back());
  auto f = as_ptrs(flag_ptrs), o = as_ptrs(out_ptrs);
  std::vector<long long> lo(seg_lo.begin(), seg_lo.end()), dst(seg_dst.begin(), seg_dst.end());
  check_rc(bdh_shard_bcast(f.data(), o.data(), out_mc, rank, world, gacc.data_ptr<float>(), (int)dst.size(), lo.data(),
                           dst.data(), scale, (unsigned)epoch, ctas, status_word().data_ptr<int>(), cur_stream()),
           "shard_bcast");
}

void decode_state_update(const Tensor& q, const Tensor& v, Tensor& rho, Tensor& a, const optional<Tensor>& slopes,
                         c10::optional<Tensor> last, const optional<Tensor>& step_dev) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(rho.dim() == 4 && rho.is_contiguous() && rho.scalar_type() == at::kFloat);
  const int64_t B = rho.size(0), H = rho.size(1), Np = rho.size(2), D = rho.size(3);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && q.is_contiguous() && q.numel() == B * H * Np);
  TORCH_CHECK(v.scalar_type() == at::kBFloat16 && v.is_contiguous() && v.numel() == B * D);
  TORCH_CHECK(a.scalar_type() == at::kFloat && a.is_contiguous() && a.numel() == H * B * D);
  TORCH_CHECK(last.has_value() == step_dev.has_value(), "decode_state_update: last and step_dev come together");
  if (last.has_value())
    TORCH_CHECK(last->is_cuda() && last->is_contiguous() && last->scalar_type() == at::kInt && last->numel() == B * H * Np &&
                step_dev->is_cuda() && step_dev->scalar_type() == at::kInt && step_dev->numel() >= 1 && slopes.has_value(),
                "decode_state_update: last int32 [B,H,Np], step_dev int32 [1], with slopes");
  check_rc(bdh_decode_state_update(q.data_ptr(), v.data_ptr(), rho.data_ptr<float>(), a.data_ptr<float>(),
                                   slopes.has_value() ? slopes->data_ptr<float>() : nullptr,
                                   last.has_value() ? last->data_ptr<int>() : nullptr,
                                   step_dev.has_value() ? step_dev->data_ptr<int>() : nullptr, B, H, Np, D, cur_stream()),
           "decode_state_update");
}
void sample_tokens(const Tensor& logits, Tensor& out, double temperature, int64_t top_k, bool greedy, int64_t seed,
                   int64_t step, const optional<Tensor>& step_dev) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kFloat);
  TORCH_CHECK(out.scalar_type() == at::kLong && out.is_contiguous() && out.numel() == logits.size(0));
  check_rc(bdh_sample_tokens(logits.data_ptr<float>(), reinterpret_cast<long long*>(out.data_ptr<int64_t>()),
                             logits.size(0), logits.size(1), temperature, top_k, greedy, (unsigned)seed,
                             step_dev.has_value() ? step_dev->data_ptr<int>() : nullptr, step, cur_stream()),
           "sample_tokens");
}
void viz_encode_units(const Tensor& values, Tensor& image, int64_t cursor, int64_t row0, double gain,
                      at::ArrayRef<double> lo, at::ArrayRef<double> hi, at::ArrayRef<double> sep, int64_t units_per_head) {
  c10::cuda::CUDAGuard guard(values.device());
  TORCH_CHECK(values.scalar_type() == at::kFloat && values.is_contiguous());
  TORCH_CHECK(image.scalar_type() == at::kFloat && image.is_contiguous() && image.dim() == 3 && image.size(2) == 4 &&
              row0 + values.numel() <= image.size(0) && lo.size() == 3 && hi.size() == 3 && sep.size() == 3);
  float l[3] = {(float)lo[0], (float)lo[1], (float)lo[2]}, h[3] = {(float)hi[0], (float)hi[1], (float)hi[2]};
  float sp[3] = {(float)sep[0], (float)sep[1], (float)sep[2]};
  check_rc(bdh_viz_encode_units(values.data_ptr<float>(), image.data_ptr<float>(), values.numel(), image.size(1), cursor,
                                row0, gain, l, h, sp, units_per_head, cur_stream()), "viz_encode_units");
}
void rope_table_step(const Tensor& pos, const Tensor& pair_freqs, Tensor& table) {
  c10::cuda::CUDAGuard guard(pos.device());
  TORCH_CHECK(pos.scalar_type() == at::kInt && pair_freqs.scalar_type() == at::kFloat && pair_freqs.is_contiguous());
  TORCH_CHECK(table.is_contiguous() && table.element_size() == 2 && table.numel() == 2 * pair_freqs.numel());
  check_rc(bdh_rope_table_step(pos.data_ptr<int>(), pair_freqs.data_ptr<float>(), table.data_ptr(), pair_freqs.numel(),
                               cur_stream()), "rope_table_step");
}
void bump_counter(Tensor& counter, int64_t by) {
  c10::cuda::CUDAGuard guard(counter.device());
  TORCH_CHECK(counter.scalar_type() == at::kInt);
  check_rc(bdh_bump_counter(counter.data_ptr<int>(), by, cur_stream()), "bump_counter");
}

static void check_f32(std::initializer_list<const Tensor*> ts) {
  for (const Tensor* t : ts)
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat, "expected contiguous fp32 CUDA tensors");
}

void conv1d_silu_fwd(const Tensor& seq, const Tensor& w, const c10::optional<Tensor>& bias, Tensor& out) {
  c10::cuda::CUDAGuard guard(seq.device());
  check_f32({&seq, &w, &out});
  if (bias.has_value()) check_f32({&*bias});
  const int64_t B = out.size(0), T = out.size(1), C = out.size(2), k = w.size(1);
  TORCH_CHECK(seq.dim() == 3 && out.dim() == 3 && w.dim() == 2 && w.size(0) == C && seq.size(0) == B &&
              seq.size(1) == T + k - 1 && seq.size(2) == C && (!bias.has_value() || bias->numel() == C), "conv1d_silu_fwd: shapes");
  check_rc(bdh_conv1d_silu_fwd(seq.data_ptr<float>(), w.data_ptr<float>(), bias.has_value() ? bias->data_ptr<float>() : nullptr,
                               out.data_ptr<float>(), B, T, C, k, cur_stream()), "conv1d_silu_fwd");
}

void conv1d_silu_bwd(const Tensor& seq, const Tensor& w, const c10::optional<Tensor>& bias, const Tensor& dout, Tensor& dpre,
                     Tensor& dseq, Tensor& dw, c10::optional<Tensor> db) {
  c10::cuda::CUDAGuard guard(seq.device());
  check_f32({&seq, &w, &dout, &dpre, &dseq, &dw});
  if (bias.has_value()) check_f32({&*bias});
  if (db.has_value()) check_f32({&*db});
  const int64_t B = dout.size(0), T = dout.size(1), C = dout.size(2), k = w.size(1);
  TORCH_CHECK(seq.dim() == 3 && dout.dim() == 3 && w.dim() == 2 && w.size(0) == C && seq.size(0) == B &&
              seq.size(1) == T + k - 1 && seq.size(2) == C && dpre.numel() == dout.numel() && dseq.numel() == seq.numel() &&
              dw.numel() == w.numel() && (!db.has_value() || db->numel() == C), "conv1d_silu_bwd: shapes");
  check_rc(bdh_conv1d_silu_bwd(seq.data_ptr<float>(), w.data_ptr<float>(), bias.has_value() ? bias->data_ptr<float>() : nullptr,
                               dout.data_ptr<float>(), dpre.data_ptr<float>(), dseq.data_ptr<float>(), dw.data_ptr<float>(),
                               db.has_value() ? db->data_ptr<float>() : nullptr, B, T, C, k, cur_stream()), "conv1d_silu_bwd");
}

void gated_rmsnorm_fwd(const Tensor& v, const Tensor& z, const Tensor& w, Tensor& out, Tensor& rstd, double eps) {
  c10::cuda::CUDAGuard guard(v.device());
  check_f32({&v, &z, &w, &out, &rstd});
  const int64_t D = v.size(-1), rows = v.numel() / D;
  TORCH_CHECK(z.numel() == v.numel() && out.numel() == v.numel() && w.numel() == D && rstd.numel() == rows, "gated_rmsnorm_fwd: shapes");
  check_rc(bdh_gated_rmsnorm_fwd(v.data_ptr<float>(), z.data_ptr<float>(), w.data_ptr<float>(), out.data_ptr<float>(),
                                 rstd.data_ptr<float>(), rows, D, static_cast<float>(eps), cur_stream()), "gated_rmsnorm_fwd");
}

void gated_rmsnorm_bwd(const Tensor& v, const Tensor& z, const Tensor& w, const Tensor& rstd, const Tensor& dout, Tensor& dv,
                       Tensor& dz, Tensor& dw) {
  c10::cuda::CUDAGuard guard(v.device());
  check_f32({&v, &z, &w, &rstd, &dout, &dv, &dz, &dw});
  const int64_t D = v.size(-1), rows = v.numel() / D;
  TORCH_CHECK(z.numel() == v.numel() && dout.numel() == v.numel() && dv.numel() == v.numel() && dz.numel() == v.numel() &&
              w.numel() == D && dw.numel() == D && rstd.numel() == rows, "gated_rmsnorm_bwd: shapes");
  check_rc(bdh_gated_rmsnorm_bwd(v.data_ptr<float>(), z.data_ptr<float>(), w.data_ptr<float>(), rstd.data_ptr<float>(),
                                 dout.data_ptr<float>(), dv.data_ptr<float>(), dz.data_ptr<float>(), dw.data_ptr<float>(), rows, D,
                                 cur_stream()), "gated_rmsnorm_bwd");
}

void ssd_decode_step(const Tensor& xw, const Tensor& loga, const Tensor& Bm, const Tensor& Cm, Tensor& h, Tensor& y) {
  c10::cuda::CUDAGuard guard(xw.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&xw, &loga, &Bm, &Cm, &h, &y})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat);
  const int64_t B = xw.size(0), H = xw.size(1);
  TORCH_CHECK(xw.dim() == 3 && xw.size(2) == 64 && Bm.numel() == B * 128 && Cm.numel() == B * 128 && loga.numel() == B * H &&
              h.numel() == B * H * 128 * 64 && y.numel() == xw.numel());
  check_rc(bdh_ssd_decode_step(xw.data_ptr<float>(), loga.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(),
                               h.data_ptr<float>(), y.data_ptr<float>(), B, H, cur_stream()), "ssd_decode_step");
}

void ssd_chunk_scan(const Tensor& xw, const Tensor& loga, const Tensor& Bm, const Tensor& Cm, Tensor& h, Tensor& states,
                    Tensor& decay, Tensor& y, bool tensor_cores) {
  c10::cuda::CUDAGuard guard(xw.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&xw, &loga, &Bm, &Cm, &h, &states, &decay, &y})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kFloat);
  const int64_t B = xw.size(0), T = xw.size(1), H = xw.size(2);
  TORCH_CHECK(xw.size(3) == 64 && Bm.size(2) == 128 && Cm.size(2) == 128 && T % 64 == 0);
  TORCH_CHECK(h.numel() == B * H * 128 * 64 && y.numel() == xw.numel() && states.numel() == B * (T / 64) * H * 128 * 64 &&
              decay.numel() == B * (T / 64) * H);
  if (tensor_cores) {
    check_rc(bdh_ssd_chunk_scan_tc(xw.data_ptr<float>(), loga.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(),
                                   h.data_ptr<float>(), states.data_ptr<float>(), decay.data_ptr<float>(),
                                   y.data_ptr<float>(), B, T, H, status_word().data_ptr<int>(), cur_stream()),
             "ssd_chunk_scan_tc");
    return;
  }
  check_rc(bdh_ssd_chunk_scan(xw.data_ptr<float>(), loga.data_ptr<float>(), Bm.data_ptr<float>(), Cm.data_ptr<float>(),
                              h.data_ptr<float>(), states.data_ptr<float>(), decay.data_ptr<float>(), y.data_ptr<float>(),
                              B, T, H, cur_stream()), "ssd_chunk_scan");
}

void graph_spmm_relu(const Tensor& x, const Tensor& w, const Tensor& ell, Tensor& y, double theta) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1) && x.is_contiguous() && w.is_contiguous());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16);
  TORCH_CHECK(ell.scalar_type() == at::kInt && ell.is_contiguous() && ell.dim() == 2 && ell.size(0) == (w.size(0) + 63) / 64);
  TORCH_CHECK(y.is_contiguous() && y.size(0) == x.size(0) && y.size(1) == w.size(0));
  check_rc(bdh_graph_spmm_relu(x.data_ptr(), w.data_ptr(), ell.data_ptr<int>(), y.data_ptr(), x.size(0), w.size(0), x.size(1),
                               ell.size(1), theta, cur_stream()), "graph_spmm_relu");
}

void rank_barrier(const Tensor& anchor, at::IntArrayRef flag_ptrs, int64_t rank, int64_t world, int64_t epoch) {
  c10::cuda::CUDAGuard guard(anchor.device());
  auto f = as_ptrs(flag_ptrs);
  check_rc(bdh_rank_barrier(f.data(), rank, world, (unsigned)epoch, status_word().data_ptr<int>(), cur_stream()),
           "rank_barrier");
}

void pope_bwd(const Tensor& dq, const Tensor& x, const Tensor& dxg, const Tensor& freqs, Tensor& dx, int64_t H, int64_t T,
              int64_t pos0) {
  c10::cuda::CUDAGuard guard(x.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&dq, &x, &dxg, &dx})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kBFloat16 && t->dim() == 2);
  const int64_t M = x.size(0), HN = x.size(1);
  TORCH_CHECK(HN % H == 0 && dq.size(0) == M && dq.size(1) == 2 * HN && dxg.sizes() == x.sizes() && dx.sizes() == x.sizes());
  TORCH_CHECK(freqs.scalar_type() == at::kFloat && freqs.is_contiguous() && freqs.numel() == HN / H);
  check_rc(bdh_pope_bwd(dq.data_ptr(), x.data_ptr(), dxg.data_ptr(), freqs.data_ptr<float>(), dx.data_ptr(), M, H, HN / H, T,
                        pos0, cur_stream()), "pope_bwd");
}

void state_scan(const Tensor& seg, const optional<Tensor>& start, const optional<Tensor>& decay, Tensor& out16,
                c10::optional<Tensor> total, int64_t J, int64_t H, bool backward) {
  c10::cuda::CUDAGuard guard(seg.device());
  TORCH_CHECK(seg.is_cuda() && seg.is_contiguous() && seg.scalar_type() == at::kFloat, "seg: contiguous fp32");
  TORCH_CHECK(out16.is_cuda() && out16.is_contiguous() && out16.scalar_type() == at::kBFloat16 && out16.numel() == seg.numel());
  TORCH_CHECK(J >= 1 && H >= 1 && seg.numel() % (J * H) == 0);
  const int64_t D = seg.size(-1), rows = seg.numel() / D;              // [B*J*H*Np, D] or any view of it
  (void)rows;
  // per = N' * D elements per (b, j, h): the caller passes seg as [B*J, H, Np, D]
  TORCH_CHECK(seg.dim() == 4 && seg.size(1) == H && seg.size(0) % J == 0, "seg: [B*J, H, Np, D]");
  const int64_t per = seg.size(2) * seg.size(3), n_bh = seg.size(0) / J * H;
  for (const optional<Tensor>* t : {&start, static_cast<const optional<Tensor>*>(&total)})
    if (t->has_value())
      TORCH_CHECK((*t)->is_cuda() && (*t)->is_contiguous() && (*t)->scalar_type() == at::kFloat && (*t)->numel() == n_bh * per);
  if (decay.has_value())
    TORCH_CHECK(decay->is_cuda() && decay->is_contiguous() && decay->scalar_type() == at::kFloat && decay->numel() == H);
  check_rc(bdh_state_scan(seg.data_ptr<float>(), start.has_value() ? start->data_ptr<float>() : nullptr,
                          decay.has_value() ? decay->data_ptr<float>() : nullptr, out16.data_ptr(),
                          total.has_value() ? total->data_ptr<float>() : nullptr, per, J, H, n_bh, backward ? 1 : 0,
                          cur_stream()), "state_scan");
}

void pope_rotate(const Tensor& x, const Tensor& freqs, Tensor& q, int64_t H, int64_t T, int64_t pos0) {
  c10::cuda::CUDAGuard guard(x.device());
  for (const Tensor* t : std::initializer_list<const Tensor*>{&x, &q})
    TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == at::kBFloat16 && t->dim() == 2);
  const int64_t M = x.size(0), HN = x.size(1);
  TORCH_CHECK(HN % H == 0 && q.size(0) == M && q.size(1) == 2 * HN);
  TORCH_CHECK(freqs.scalar_type() == at::kFloat && freqs.is_contiguous() && freqs.numel() == HN / H);
  check_rc(bdh_pope_rotate(x.data_ptr(), freqs.data_ptr<float>(), q.data_ptr(), M, H, HN / H, T, pos0, cur_stream()),
           "pope_rotate");
}

void wait_timeout_probe(const Tensor& flag, int64_t value, int64_t limit_ns) {
  c10::cuda::CUDAGuard guard(flag.device());
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt);
  check_rc(bdh_wait_timeout_probe(reinterpret_cast<const unsigned*>(flag.data_ptr<int>()), (unsigned)value,
                                  (unsigned long long)limit_ns, status_word().data_ptr<int>(), cur_stream()),
           "wait_timeout_probe");
}

}  // namespace

TORCH_LIBRARY(bdh, m) {
  m.def("gemm(Tensor a, bool a_mn, Tensor b, bool b_mn, int M, int N, int K, int nz0, int nz1, int[] a_off, "
        "int[] b_off, int epi, int flags, Tensor(a!)? out0, Tensor(b!)? out1, Tensor? in0, Tensor? in1, "
        "int[] c_off, int[] o1_off, float alpha, float theta, int T, int pos0, int n_per_head, "
        "Tensor? freqs, Tensor? slopes, int causal_tiles, int causal_k, int bn, int max_ctas, bool tma_epilogue, int mc_out, float drop_p, int drop_seed, int[] peer_ptrs, int peer_rows, int peer_rank, Tensor? bias, "
        "int[] gather_ptrs, int gather_rows, int gather_rank, Tensor(c!)? gather_arrived, Tensor? tile_skip) -> ()");
  m.def("dual_gemm(Tensor a1, Tensor b1, bool b1_mn, Tensor b2, Tensor(a!) p, int M, int H, int n_per_head, int K1, int N2, "
        "int T, int epi, int flags, int group_per_head, int a1_b, int a1_h, int b1_b, Tensor? in0, Tensor? in1, "
        "Tensor(b!)? out1, float alpha, float theta, int pos0, float drop_p, int drop_seed, Tensor(c!) partials, "
        "int max_ctas) -> ()");
  m.def("dual_gemm_reduce(Tensor partials, int M, int H, int n_per_head, int N2, int group_per_head, int max_ctas, "
        "Tensor(a!) out, bool accumulate, int out_h_stride) -> ()");
  m.def("dual_gemm_partial_floats(int M, int H, int n_per_head, int N2, int group_per_head, int max_ctas) -> int");
  m.def("layernorm_fwd(Tensor x, Tensor(a!) y) -> ()");
  m.def("layernorm_bwd(Tensor x, Tensor dy, Tensor(a!) dx, bool accumulate) -> ()");
  m.def("embed_ln_fwd(Tensor tokens, Tensor emb, Tensor(a!) cur) -> ()");
  m.def("embed_ln_bwd(Tensor tokens, Tensor emb, Tensor dcur, Tensor(a!) demb) -> ()");
  m.def("block_out_fwd(Tensor cur, Tensor mlp, Tensor(a!) out) -> ()");
  m.def("layernorm_f32_clear(Tensor(a!) a, Tensor(b!) y) -> ()");
  m.def("block_out_parts(Tensor cur, Tensor part, Tensor(a!) out) -> ()");
  m.def("block_out_bwd(Tensor cur, Tensor mlp, Tensor dout, Tensor(a!) dcur, Tensor(b!) dmlp) -> ()");
  m.def("cross_entropy(Tensor logits, Tensor targets, Tensor(a!) row_loss, Tensor(b!)? dlogits, float grad_scale) -> ()");
  m.def("adamw(Tensor(a!) master, Tensor grad, Tensor(b!) m, Tensor(c!) v, Tensor(d!)? p16, float lr, float beta1, "
        "float beta2, float eps, float wd, int step, float grad_scale) -> ()");
  m.def("status() -> Tensor");
  m.def("bounds_records(bool clear) -> Tensor");
  m.def("rownorm_fwd(Tensor(a!) scores, Tensor(b!) rnorm, int T) -> ()");
  m.def("rownorm_bwd(Tensor(a!) grad, Tensor normed, Tensor rnorm, int T) -> ()");
  m.def("allreduce_scale(Tensor anchor, int[] buf_ptrs, int[] flag_ptrs, int mc_ptr, int rank, int world, "
        "int n_floats, float scale, int epoch, int ctas) -> ()");
  m.def("gather_blocks(Tensor anchor, int[] slot_ptrs, int[] flag_ptrs, int[] out_ptrs, int out_mc, bool out_bf16, "
        "int rank, int world, int block_floats, int epoch, int ctas) -> ()");
  m.def("rs_adamw_ag(Tensor anchor, int[] grad_ptrs, int[] flag_ptrs, int grad_mc, int[] shadow_ptrs, int rank, "
        "int world, int n_floats, Tensor(a!) master, Tensor(b!) m, Tensor(c!) v, float lr, float beta1, "
        "float beta2, float eps, float wd, int step, float grad_scale, int epoch, int ctas) -> ()");
  m.def("shard_adamw_ag(int[] flag_ptrs, int[] shadow_ptrs, int rank, int world, Tensor(a!) gacc, Tensor(b!) master, "
        "Tensor(c!) m, Tensor(d!) v, int[] seg_lo, int[] seg_dst, float lr, float beta1, float beta2, float eps, "
        "float wd, int step, float grad_scale, int epoch, int ctas) -> ()");
  m.def("shard_bcast(int[] flag_ptrs, int[] out_ptrs, int out_mc, int rank, int world, Tensor(a!) gacc, int[] seg_lo, "
        "int[] seg_dst, float scale, int epoch, int ctas) -> ()");
  m.def("wait_timeout_probe(Tensor flag, int value, int limit_ns) -> ()");
  m.def("pope_bwd(Tensor dq, Tensor x, Tensor dxg, Tensor freqs, Tensor(a!) dx, int H, int T, int pos0) -> ()");
  m.def("pope_rotate(Tensor x, Tensor freqs, Tensor(a!) q, int H, int T, int pos0) -> ()");
  m.def("state_scan(Tensor seg, Tensor? start, Tensor? decay, Tensor(a!) out16, Tensor(b!)? total, int J, int H, bool backward) -> ()");
  m.def("rank_barrier(Tensor anchor, int[] flag_ptrs, int rank, int world, int epoch) -> ()");
  m.def("graph_spmm_relu(Tensor x, Tensor w, Tensor ell, Tensor(a!) y, float theta) -> ()");
  m.def("ssd_decode_step(Tensor xw, Tensor loga, Tensor Bm, Tensor Cm, Tensor(a!) h, Tensor(b!) y) -> ()");
  m.def("conv1d_silu_fwd(Tensor seq, Tensor w, Tensor? bias, Tensor(a!) out) -> ()");
  m.def("conv1d_silu_bwd(Tensor seq, Tensor w, Tensor? bias, Tensor dout, Tensor(a!) dpre, Tensor(b!) dseq, Tensor(c!) dw, "
        "Tensor(d!)? db) -> ()");
  m.def("gated_rmsnorm_fwd(Tensor v, Tensor z, Tensor w, Tensor(a!) out, Tensor(b!) rstd, float eps) -> ()");
  m.def("gated_rmsnorm_bwd(Tensor v, Tensor z, Tensor w, Tensor rstd, Tensor dout, Tensor(a!) dv, Tensor(b!) dz, "
        "Tensor(c!) dw) -> ()");
  m.def("ssd_chunk_scan(Tensor xw, Tensor loga, Tensor Bm, Tensor Cm, Tensor(a!) h, Tensor(b!) states, Tensor(c!) decay, "
        "Tensor(d!) y, bool tensor_cores) -> ()");
  m.def("decode_state_update(Tensor q, Tensor v, Tensor(a!) rho, Tensor(b!) a, Tensor? slopes, Tensor(c!)? last=None, "
        "Tensor? step_dev=None) -> ()");
  m.def("sample_tokens(Tensor logits, Tensor(a!) out, float temperature, int top_k, bool greedy, int seed, int step, "
        "Tensor? step_dev) -> ()");
  m.def("viz_encode_units(Tensor values, Tensor(a!) image, int cursor, int row0, float gain, float[] lo, float[] hi, "
        "float[] sep, int units_per_head) -> ()");
  m.def("rope_table_step(Tensor pos, Tensor pair_freqs, Tensor(a!) table) -> ()");
  m.def("bump_counter(Tensor(a!) counter, int by) -> ()");
}

TORCH_LIBRARY_IMPL(bdh, CUDA, m) {
  m.impl("gemm", &gemm);
  m.impl("dual_gemm", &dual_gemm);
  m.impl("dual_gemm_reduce", &dual_gemm_reduce);
  m.impl("layernorm_fwd", &layernorm_fwd);
  m.impl("layernorm_bwd", &layernorm_bwd);
  m.impl("embed_ln_fwd", &embed_ln_fwd);
  m.impl("embed_ln_bwd", &embed_ln_bwd);
  m.impl("block_out_fwd", &block_out_fwd);
  m.impl("layernorm_f32_clear", &layernorm_f32_clear);
  m.impl("block_out_parts", &block_out_parts);
  m.impl("block_out_bwd", &block_out_bwd);
  m.impl("cross_entropy", &cross_entropy);
  m.impl("adamw", &adamw);
  m.impl("rownorm_fwd", &rownorm_fwd);
  m.impl("rownorm_bwd", &rownorm_bwd);
  m.impl("allreduce_scale", &allreduce_scale);
  m.impl("gather_blocks", &gather_blocks);
  m.impl("rs_adamw_ag", &rs_adamw_ag);
  m.impl("shard_adamw_ag", &shard_adamw_ag);
  m.impl("shard_bcast", &shard_bcast);
  m.impl("wait_timeout_probe", &wait_timeout_probe);
  m.impl("pope_bwd", &pope_bwd);
  m.impl("pope_rotate", &pope_rotate);
  m.impl("state_scan", &state_scan);
  m.impl("rank_barrier", &rank_barrier);
  m.impl("graph_spmm_relu", &graph_spmm_relu);
  m.impl("ssd_decode_step", &ssd_decode_step);
  m.impl("conv1d_silu_fwd", &conv1d_silu_fwd);
  m.impl("conv1d_silu_bwd", &conv1d_silu_bwd);
  m.impl("gated_rmsnorm_fwd", &gated_rmsnorm_fwd);
  m.impl("gated_rmsnorm_bwd", &gated_rmsnorm_bwd);
  m.impl("ssd_chunk_scan", &ssd_chunk_scan);
  m.impl("decode_state_update", &decode_state_update);
  m.impl("sample_tokens", &sample_tokens);
  m.impl("viz_encode_units", &viz_encode_units);
  m.impl("rope_table_step", &rope_table_step);
  m.impl("bump_counter", &bump_counter);
}
TORCH_LIBRARY_IMPL(bdh, CompositeExplicitAutograd, m) {
  m.impl("status", &status);
  m.impl("dual_gemm_partial_floats", &dual_gemm_partial_floats);
  m.impl("bounds_records", &bounds_records);
}
