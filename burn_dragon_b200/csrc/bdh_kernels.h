// C interface of the sm_100a kernels. Everything here takes raw device pointers and a stream,
// allocates nothing and returns a BDH_* code; the torch binding (bindings.cpp) is one caller,
// any C/C++ program that links the library is another.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  BDH_OK = 0,
  BDH_ERR_DRIVER = 1,       // could not resolve a driver entry point
  BDH_ERR_ALIGNMENT = 2,    // pointer not 16-byte aligned or leading dimension not a multiple of 8
  BDH_ERR_TMAP = 3,         // tensor-map encoding rejected the matrix
  BDH_ERR_LAUNCH = 4,
  BDH_ERR_ARGUMENT = 5,
  BDH_ERR_UNSUPPORTED = 6,  // no kernel instantiation for this (majors, epilogue, tile)
  BDH_ERR_TOO_LARGE = 7,
};

// bf16 row-major 2-D matrix view: element (r, c) at ptr[r*ld + c].
typedef struct {
  const void* ptr;
  long long rows, cols, ld;
} BdhMat;

// One batched GEMM  C[z][m,n] = epi(sum_k A[z][m,k] B[z][n,k]),  z = (z0, z1).
// a_off/b_off = {mn per z0, mn per z1, k per z0, k per z1} element offsets into the 2-D views;
// c_off = {row per z0, row per z1, col per z0, col per z1}; o1_off = {col per z0, col per z1,
// imag distance} for the second output of the rotary epilogue.
typedef struct {
  int M, N, K, nz0, nz1;
  long long a_off[4], b_off[4], c_off[4], o1_off[3];
  int epi, flags, bn;
  int causal_tiles, causal_k;
  void* out0;
  void* out1;
  const void* in0;
  const void* in1;
  long long ld_out0, ld_out1, ld_in0, ld_in1;
  float alpha, theta;
  int T, pos0, n_per_head;
  const float* freqs;
  const float* slopes;
  const float* bias;   // epi 1 / 2: fp32 bias per output column, added before the threshold (16-byte aligned; nullptr: none)
  int* status;   // device word that receives a STATUS_* code if an in-kernel wait gives up
  int max_ctas;  // 0: one CTA per SM
  int no_tma_epilogue;  // 1: force the per-thread global-memory epilogue
  float drop_p;         // EPI_RELU_GATE: dropout probability on x*y
  unsigned drop_seed;
  // Reduce-scatter epilogue (flag 1024, fp32 EPI_STORE): peer_out[r] is rank r's mapping of the
  // symmetric slot buffer [peer_world][peer_rows][ld_out0]; output rows [r*peer_rows, (r+1)*peer_rows)
  // are stored into slot peer_rank of rank r's buffer.
  const long long* peer_out;
  int peer_world, peer_rank;
  long long peer_rows;
  // All-gather of A inside the kernel (gather_world > 1): A is this rank's copy of a symmetric contiguous
  // [M, K] bf16 buffer of which every rank has written its own gather_rows rows (M = gather_world * gather_rows,
  // gather_rows % 128 == 0); gather_src[r] is rank r's copy. The kernel pulls the other ranks' rows into A with
  // peer loads and starts a row block's tiles once it has arrived; gather_arrived holds M / 128 zeroed counters.
  // K-major A, one problem (nz0 = nz1 = 1). The caller orders the launch after every rank's writes (a rank
  // barrier before) and keeps the rows unchanged until every rank's launch is over (a rank barrier after).
  // Causal epilogue only: [ceil(M/128), ceil(N/bn)] bytes, non-zero = skip this output tile (nullptr: none).
  const unsigned char* tile_skip;
  const long long* gather_src;
  int gather_world, gather_rank;
  long long gather_rows;
  unsigned* gather_arrived;
} BdhGemmDesc;

int bdh_gemm_bf16(const BdhMat* A, int a_mn_major, const BdhMat* B, int b_mn_major,
                  const BdhGemmDesc* desc, cudaStream_t stream);

// ---- two chained GEMMs with the [tokens, neurons] intermediate kept on chip (dual_gemm_sm100.cu) ----
//   Y = A1 . B1^T  (per 128-token tile and 128-neuron chunk; contraction length K1)
//   P = epilogue(Y; in0, in1)  -> written once to the bf16 matrix P [M, H*n_per_head] (and out1)
//   OUT[group] = sum over the group's chunks of P . B2   (B2 [H*n_per_head, N2] bf16, N2 <= 256)
// epi 2 (ReLU + gate): P = relu(Y - theta) * in0 (dropout as in bdh_gemm_bf16);
// epi 4 (gate backward): in0 = x, in1 = x*y, P = d y, out1 = gate gradient w.r.t. x (marked);
// epi 5 (rotation backward): in0 = marked gate gradient, in1 = rotary table, P = d x.
// A1 row of (token tile mt, head h) = (mt / (T/128)) * a1_b + (mt % (T/128)) * 128 + h * a1_h.
// b1_mn = 1: B1 is indexed [k, neuron] and the k rows of tile mt start at (mt / (T/128)) * b1_b.
// group_per_head = 0: OUT is [M, N2], summed over all heads; 1: one [M, N2] block per head.
// The sums arrive as fp32 partial tiles in `partials` (size from bdh_dual_gemm_partial_floats);
// bdh_dual_gemm_reduce, given the same descriptor, adds them up in a fixed order into `out`
// (row of head h, token m: h * out_h_stride + m), as bf16, fp32 or fp32 +=.
typedef struct {
  int M, H, n_per_head, K1, N2, T;
  int epi, flags, group_per_head;
  long long a1_b, a1_h, b1_b;
  const void* in0;
  const void* in1;
  void* out1;
  long long ld_in0, ld_in1, ld_out1;
  float alpha, theta;
  int pos0;
  float drop_p;
  unsigned drop_seed;
  float* partials;
  long long partial_floats;   // capacity of `partials`
  int* status;
  int max_ctas;               // 0: one CTA per SM
} BdhDualDesc;

long long bdh_dual_gemm_partial_floats(const BdhDualDesc* desc);
int bdh_dual_gemm(const BdhMat* A1, const BdhMat* B1, int b1_mn_major, const BdhMat* B2, const BdhMat* P,
                  const BdhDualDesc* desc, cudaStream_t stream);
int bdh_dual_gemm_reduce(const BdhDualDesc* desc, void* out, long long ld_out, int out_bf16, int accumulate,
                         long long out_h_stride, cudaStream_t stream);

// ---- row-wise kernels (rows of length D <= 2048, D % 8 == 0) ---------------------------------
// y = LayerNorm(x) without affine, eps 1e-5, biased variance (reference: src/model/bdh.rs:86-89).
int bdh_layernorm_fwd(const void* x_bf16, void* y_bf16, long long rows, int D, cudaStream_t s);
// dx (+)= LayerNorm backward given x and dy.
int bdh_layernorm_bwd(const void* x_bf16, const void* dy_bf16, void* dx_bf16, long long rows, int D,
                      int accumulate, cudaStream_t s);
// cur = LayerNorm(embedding[token]); tokens int64.
int bdh_embed_ln_fwd(const long long* tokens, const void* emb_bf16, void* cur_bf16, long long rows,
                     int D, int vocab, cudaStream_t s);
// d_emb[token] += LayerNorm backward(dcur) with fp32 atomics.
int bdh_embed_ln_bwd(const long long* tokens, const void* emb_bf16, const float* dcur_f32,
                     float* demb_f32, long long rows, int D, int vocab, cudaStream_t s);
// out = LayerNorm(cur + LayerNorm(mlp))  (reference: src/model/bdh.rs:436-441).
int bdh_block_out_fwd(const void* cur_bf16, const void* mlp_bf16, void* out_bf16, long long rows,
                      int D, cudaStream_t s);
// Decode step: y_bf16 = LayerNorm(a_f32) and a_f32 <- 0 (the rows are atomically accumulated again by the next layer).
int bdh_layernorm_f32_clear(float* a_f32, void* y_bf16, long long rows, int D, cudaStream_t s);
// Decode step: out = LayerNorm(cur + LayerNorm(sum_p part[p])) with part fp32 [parts, rows, D].
int bdh_block_out_parts(const void* cur_bf16, const float* part_f32, int parts, void* out_bf16, long long rows,
                        int D, cudaStream_t s);
// Given d_out (fp32): d_cur_f32 (=) du, d_mlp_bf16 = LNbwd(mlp, du) where u = cur + LN(mlp).
int bdh_block_out_bwd(const void* cur_bf16, const void* mlp_bf16, const float* dout_f32,
                      float* dcur_f32, void* dmlp_bf16, long long rows, int D, cudaStream_t s);

// State scans of the chunk-state attention (rowwise.cu): seg fp32 [B, J, H, per], start / total fp32 [B, H, per]
// (either may be null), decay [H] or null, out16 bf16 [B, J, H, per]. backward = 0: out16[j] = state before segment j,
// total = state after the last; backward = 1: the reverse recurrence over the gradients (see the kernel).
int bdh_state_scan(const float* seg, const float* start, const float* decay, void* out16_bf16, float* total,
                   long long per, int J, int H, long long n_bh, int backward, cudaStream_t s);
// PoPE query rebuilt from the stored x: q_bf16 [M, H*2N] (per head [real N | imag N]) = softplus(x) * (cos, sin).
int bdh_pope_rotate(const void* x_bf16, const float* freqs, void* q_bf16, long long M, int H, int N, int T, int pos0,
                    cudaStream_t s);
// PoPE backward: dx = (dq_re cos + dq_im sin) sigmoid(x) + gate gradient where x > 0, else 0.
// dq bf16 [M, H*2N] (per head [real N | imag N]); x, dxg, dx bf16 [M, H*N]; freqs [N]; N % 8 == 0.
int bdh_pope_bwd(const void* dq_bf16, const void* x_bf16, const void* dxg_bf16, const float* freqs, void* dx_bf16,
                 long long M, int H, int N, int T, int pos0, cudaStream_t s);

// L1 row normalisation of strictly causal scores S [rows, T] (row = (batch, head, t); columns
// s < t), the `forward_fast` attention (reference: src/model/attention.rs:142-175):
// forward S <- S / r with r = sum|S| + 1e-6 (stored); backward G <- (G - sign(Sn) sum(G Sn)) / r.
int bdh_rownorm_fwd(void* scores_bf16, float* rnorm, long long rows, int T, int ld, cudaStream_t s);
int bdh_rownorm_bwd(void* grad_bf16, const void* normed_bf16, const float* rnorm, long long rows, int T, int ld,
                    cudaStream_t s);

// ---- loss ------------------------------------------------------------------------------------
// Mean cross-entropy over rows of fp32 logits [rows, V] (V <= 1024); writes per-row loss and
// dlogits (bf16) = (softmax - onehot) * grad_scale.  (reference: src/model/loss.rs:5-18)
int bdh_cross_entropy(const float* logits, const long long* targets, float* row_loss,
                      void* dlogits_bf16, long long rows, int V, float grad_scale, cudaStream_t s);

// ---- optimizer -------------------------------------------------------------------------------
// Decoupled-weight-decay Adam over a flat fp32 master buffer; also refreshes the bf16 copy.
int bdh_adamw(float* master, const float* grad, float* m, float* v, void* param_bf16, long long n,
              float lr, float beta1, float beta2, float eps, float weight_decay, int step,
              float grad_scale, cudaStream_t s);

// ---- misc elementwise ------------------------------------------------------------------------
int bdh_cast_f32_to_bf16(const float* in, void* out_bf16, long long n, cudaStream_t s);
int bdh_add_f32_to_f32(const float* in, float* inout, long long n, cudaStream_t s);

// ---- cached decode (decode.cu) -------------------------------------------------------------------
// a[h*B+b,:] += sum_n q[b,h*Np+n] rho[b,h,n,:] ; rho = (rho + q^T v) * exp(-slope_h). `a` must be
// zeroed by the caller. slopes == nullptr: no decay, rows with q == 0 are skipped entirely. With slopes and
// `last` (int32 [B,H,Np]) + `step_dev` (device counter of the current step): lazy decay - row n of the stored
// state is current up to step last[n]; touched rows are caught up with exp(-slope (step - last)) and marked
// step + 1, rows with q == 0 are skipped. last == step_dev == nullptr: every row is scaled every step.
int bdh_decode_state_update(const void* q_bf16, const void* v_bf16, float* rho, float* a, const float* slopes,
                            int* last, const int* step_dev, int B, int H, int Np, int D, cudaStream_t s);
// One token per row of fp32 logits [B, V <= 1024]; step_dev (optional) is a device counter mixed
// into the random stream so a captured graph draws fresh numbers every replay.
int bdh_sample_tokens(const float* logits, long long* out, int B, int V, float temperature, int top_k,
                      int greedy, unsigned seed, const int* step_dev, int step_host, cudaStream_t s);
// Column `cursor` of an fp32 RGBA ring-buffer image [rows, history, 4] from `units` activations.
// Rows [row0, row0+units) of the image; colours are linear RGB; units_per_head > 0 draws separators.
int bdh_viz_encode_units(const float* values, float* image, int units, int history, int cursor, int row0,
                         float gain, const float* lo_rgb, const float* hi_rgb, const float* sep_rgb,
                         int units_per_head, cudaStream_t s);
// fp16 (cos, sin) pairs of the rotary phase at device-resident position *pos; and counter += by.
int bdh_rope_table_step(const int* pos, const float* pair_freqs, void* table_f16, int n_pairs, cudaStream_t s);
int bdh_bump_counter(int* counter, int by, cudaStream_t s);

// ---- SSD chunk scan for the Mamba paths (ssd.cu) -------------------------------------------------
// h_t = exp(loga_t) h_{t-1} + B_t (x) xw_t ; y_t = C_t . h_t, chunk 64, head dim 64, state dim 128.
// xw [B,T,H,64], loga [B,T,H], Bm/Cm [B,T,128], h [B,H,128,64] in/out, y [B,T,H,64]; T % 64 == 0.
// Scratch supplied by the caller: states [B,T/64,H,128,64] and decay [B,T/64,H] (fp32).
int bdh_ssd_chunk_scan(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                       float* states, float* decay, float* y, int B, int T, int H, cudaStream_t s);
// One recurrence step (cached decode): h <- exp(loga) h + B (x) xw, y = C . h. xw [B,H,64], loga [B,H],
// Bm/Cm [B,128], h [B,H,128,64] in place, y [B,H,64].
int bdh_ssd_decode_step(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h, float* y,
                        int B, int H, cudaStream_t s);
// Mamba-2 block, elementwise parts (mamba_ops.cu), fp32. Causal depthwise conv1d + bias + SiLU:
// seq [B, T + k - 1, C] (k - 1 leading rows = tail of the previous segment), w [C, k], bias [C] or null, out [B, T, C].
int bdh_conv1d_silu_fwd(const float* seq, const float* w, const float* bias, float* out, int B, int T, int C, int k,
                        cudaStream_t s);
// Backward: dpre [B, T, C] scratch, dseq [B, T + k - 1, C] written, dw [C, k] and db [C] (or null) added to.
int bdh_conv1d_silu_bwd(const float* seq, const float* w, const float* bias, const float* dout, float* dpre,
                        float* dseq, float* dw, float* db, int B, int T, int C, int k, cudaStream_t s);
// out = rmsnorm(v * silu(z)) * w over rows of D columns; rstd [rows] is kept for the backward pass.
int bdh_gated_rmsnorm_fwd(const float* v, const float* z, const float* w, float* out, float* rstd, long long rows,
                          int D, float eps, cudaStream_t s);
// dv, dz written, dw [D] added to.
int bdh_gated_rmsnorm_bwd(const float* v, const float* z, const float* w, const float* rstd, const float* dout,
                          float* dv, float* dz, float* dw, long long rows, int D, cudaStream_t s);
// The first half of the scan alone: afterwards states[b,c,h] is the state entering chunk c, h the final state.
int bdh_ssd_chunk_states(const float* xw, const float* loga, const float* Bm, float* h, float* states, float* decay,
                         int B, int T, int H, cudaStream_t s);
// Same contract as bdh_ssd_chunk_scan with the chunk outputs on the tensor cores (ssd_tc.cu: tcgen05 MMAs over
// pairs of chunks, bf16 operands, fp32 accumulation in TMEM). All pointers 16-byte aligned.
int bdh_ssd_chunk_scan_tc(const float* xw, const float* loga, const float* Bm, const float* Cm, float* h,
                          float* states, float* decay, float* y, int B, int T, int H, int* status, cudaStream_t s);

// ---- block-ELL neuron graph (graph.cu) ------------------------------------------------------------
// y[M, Ntot] = relu(x[M, D] . W[Ntot, D]^T - theta) touching only the 64x64 blocks listed in
// ell_cols [ceil(Ntot/64), ell_width] (column-block indices, -1 padded).
int bdh_graph_spmm_relu(const void* x_bf16, const void* w_bf16, const int* ell_cols, void* y_bf16, int M, int Ntot,
                        int D, int ell_width, float theta, cudaStream_t s);

// ---- NVLink collectives over symmetric memory (collectives.cu) --------------------------------
// buf_ptrs / flag_ptrs: this process's mappings of every rank's data / flag buffer (world entries);
// mc_ptr: NVSwitch multicast mapping of the data buffer or 0; n_floats % (4*world) == 0;
// `epoch` must grow by one per call on every rank; flag buffer >= ctas*world uint32, zeroed once.
int bdh_allreduce_scale(const long long* buf_ptrs, const long long* flag_ptrs, long long mc_ptr, int rank,
                        int world, long long n_floats, float scale, unsigned epoch, int ctas, int* status,
                        cudaStream_t s);
// Second half of a reduce-scatter done by GEMM epilogues (flag 1024): rank r adds up the `world`
// slots of block_floats fp32 partial sums in its slot buffer and sends the result to position
// r*block_floats of every rank's output buffer (out_ptrs / out_mc, world*block_floats elements),
// as fp32 or rounded to bf16. block_floats % 8 == 0. The reference has no multi-device path.
int bdh_gather_blocks(const long long* slot_ptrs, const long long* flag_ptrs, const long long* out_ptrs,
                      long long out_mc, int out_bf16, int rank, int world, long long block_floats,
                      unsigned epoch, int ctas, int* status, cudaStream_t s);
// Reduce-scatter of fp32 gradients + AdamW on the owned slice + all-gather of bf16 parameters.
// master / m / v hold only the owned slice (n_floats/world elements, last rank takes the remainder).
int bdh_rs_adamw_ag(const long long* grad_ptrs, const long long* flag_ptrs, long long grad_mc,
                    const long long* shadow_ptrs, int rank, int world, long long n_floats, float* master,
                    float* m, float* v, float lr, float beta1, float beta2, float eps, float wd, int step,
                    float grad_scale, unsigned epoch, int ctas, int* status, cudaStream_t s);
// Fully sharded AdamW: `gacc` is this rank's 1/world gradient slice, filled over NVLink by every rank's
// weight-gradient GEMM epilogues (flags 1024 | 512: red.add into the owner's block). The kernel waits for all
// ranks, applies AdamW to the local slices of master / m / v, writes the refreshed bf16 parameters into every
// rank's working copy (shadow_ptrs), clears gacc, and waits for all ranks again. Segment s (n_segs <= 4, one
// per sharded parameter) covers local elements [seg_lo[s], seg_lo[s+1]) and starts at bf16 element seg_dst[s]
// of the working copy; all offsets are multiples of 4.
int bdh_shard_adamw_ag(const long long* flag_ptrs, const long long* shadow_ptrs, int rank, int world, float* gacc,
                       float* master, float* m, float* v, int n_segs, const long long* seg_lo, const long long* seg_dst,
                       float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale,
                       unsigned epoch, int ctas, int* status, cudaStream_t s);
// Data-parallel gradients reduced in the weight-gradient epilogues: `gacc` is the slice this rank owns (as for
// bdh_shard_adamw_ag). After a barrier it is scaled, written to its place in every rank's full fp32 gradient
// buffer (out_ptrs / out_mc; segment s starts at element seg_dst[s]) and cleared; a second barrier follows.
int bdh_shard_bcast(const long long* flag_ptrs, const long long* out_ptrs, long long out_mc, int rank, int world,
                    float* gacc, int n_segs, const long long* seg_lo, const long long* seg_dst, float scale,
                    unsigned epoch, int ctas, int* status, cudaStream_t s);
// Device-side barrier over all ranks (bounded wait); uses slot 0 of the symmetric flag buffer.
int bdh_rank_barrier(const long long* flag_ptrs, int rank, int world, unsigned epoch, int* status, cudaStream_t s);
// Waits (at most limit_ns) for *flag to reach `value`; on expiry writes the timeout status and returns.
int bdh_wait_timeout_probe(const unsigned* flag, unsigned value, unsigned long long limit_ns, int* status,
                           cudaStream_t s);

// Checked build (-DBDH_DEBUG_BOUNDS; csrc/debug_bounds.cuh): the first data-dependent index that was
// out of range in the kernels of rowwise.cu / graph.cu. out5 = {checked build?, site, index, extent, where}.
int bdh_bounds_record_rowwise(long long* out5, int clear);
int bdh_bounds_record_graph(long long* out5, int clear);

#ifdef __cplusplus
}
#endif
