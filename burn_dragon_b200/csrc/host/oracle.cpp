// Plain C++ restatement of the canonical (recurrent) BDH forward pass, fp32 weights, double
// accumulators, one sequence (one thread per head, then per block of tokens): an oracle that
// shares no code with the torch path or the kernels,
// and the timed CPU baseline of the tiny preset. It follows the reference step by step:
//   cur_0[t]  = LN(embed[token_t])                                        src/model/bdh.rs:318-326
//   x         = relu(cur E_h - theta)                                     src/kernel/relu_lowrank.rs:7-37
//   q         = rotate(x, position t)   rope / pope / none (alibi)        src/model/attention.rs:305-349
//   a_h       = q_h . rho_h ;  rho_h = (rho_h + q_h^T v) * exp(-m_h)      src/model/bdh.rs:258-307
//   y         = relu(LN(a) E_v,h - theta) ;  xy = x * y                   src/model/bdh.rs:412-430
//   cur_{l+1} = LN(cur_l + LN(xy D))                                      src/model/bdh.rs:436-441
//   logits    = cur_L lm_head                                             src/model/bdh.rs:447-449
// LayerNorm is affine-free with eps 1e-5 and biased variance (src/model/bdh.rs:17,86-89); all L
// layers share the same weights. Weights use this framework's neuron-major layout:
// encoder / encoder_v / decoder are [H*N, D], embed is [V, D], lm_head is [D, V].
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

namespace {

void layer_norm(const double* x, double* y, int n) {
  double mean = 0.0;
  for (int i = 0; i < n; ++i) mean += x[i];
  mean /= n;
  double var = 0.0;
  for (int i = 0; i < n; ++i) var += (x[i] - mean) * (x[i] - mean);
  var /= n;
  const double inv = 1.0 / std::sqrt(var + 1e-5);
  for (int i = 0; i < n; ++i) y[i] = (x[i] - mean) * inv;
}

double softplus(double v) { return v > 20.0 ? v : std::log1p(std::exp(v)); }

}  // namespace

extern "C" {

// rotary: 0 = none (ALiBi: the state decays by exp(-slopes[h]) per step), 1 = rope, 2 = pope.
// freqs [N]: cycles per position for every neuron of a head (rope: equal within a pair).
// slopes [H] (used only when rotary == 0). rho_out (optional): final state of the LAST layer,
// [H, N', D] with N' = 2N for pope. Returns 0, or -1 on a bad argument.
int bdh_oracle_forward(const float* embed, const float* encoder, const float* encoder_v, const float* decoder,
                       const float* lm_head, const float* freqs, const float* slopes, const int64_t* tokens,
                       int T, int L, int D, int H, int N, int V, int rotary, float relu_threshold, int pos0,
                       float* logits, double* rho_out) {
  if (T < 1 || L < 1 || D < 1 || H < 1 || N < 1 || V < 1 || rotary < 0 || rotary > 2) return -1;
  if (rotary == 1 && (N & 1)) return -1;
  const int Np = rotary == 2 ? 2 * N : N;
  const double two_pi = 6.283185307179586476925287;
  std::vector<double> cur(static_cast<size_t>(T) * D), nxt(static_cast<size_t>(T) * D);
  std::vector<double> tmp(D);
  for (int t = 0; t < T; ++t) {
    const int64_t tok = tokens[t];
    if (tok < 0 || tok >= V) return -1;
    for (int d = 0; d < D; ++d) tmp[d] = embed[tok * D + d];
    layer_norm(tmp.data(), &cur[static_cast<size_t>(t) * D], D);
  }
  // Per layer, the heads are independent over the whole sequence (each owns its state); only the
  // decoder sum joins them, per token. So: phase A runs one thread per head over all tokens and
  // leaves x*y in `xy_all`; phase B runs over blocks of tokens. The arithmetic and its order are
  // those of the single-threaded statement, so the result does not depend on the thread count.
  std::vector<double> xy_all(static_cast<size_t>(T) * H * N);
  const int hw = static_cast<int>(std::max(1u, std::thread::hardware_concurrency()));
  for (int l = 0; l < L; ++l) {
    auto head_pass = [&](int h) {
      std::vector<double> xh(N), q(Np), a(D), lna(D);
      std::vector<double> r(static_cast<size_t>(Np) * D, 0.0);
      const double decay = rotary == 0 ? std::exp(-static_cast<double>(slopes[h])) : 1.0;
      for (int t = 0; t < T; ++t) {
        const double* c = &cur[static_cast<size_t>(t) * D];
        const double pos = static_cast<double>(pos0 + t);
        for (int n = 0; n < N; ++n) {
          const float* w = encoder + (static_cast<size_t>(h) * N + n) * D;
          double s = 0.0;
          for (int d = 0; d < D; ++d) s += c[d] * w[d];
          s -= relu_threshold;
          xh[n] = s > 0.0 ? s : 0.0;
        }
        // positional rotation of the query / key
        if (rotary == 0) {
          for (int n = 0; n < N; ++n) q[n] = xh[n];
        } else if (rotary == 1) {
          for (int n = 0; n < N; n += 2) {
            const double raw = pos * static_cast<double>(freqs[n]);
            const double ph = (raw - std::floor(raw)) * two_pi;
            const double co = std::cos(ph), si = std::sin(ph);
            q[n] = xh[n] * co - xh[n + 1] * si;
            q[n + 1] = xh[n + 1] * co + xh[n] * si;
          }
        } else {
          for (int n = 0; n < N; ++n) {
            const double raw = pos * static_cast<double>(freqs[n]);
            const double ph = (raw - std::floor(raw)) * two_pi;
            const double mag = softplus(xh[n]);
            q[n] = mag * std::cos(ph);
            q[N + n] = mag * std::sin(ph);
          }
        }
        // a = q . rho ; rho = (rho + q^T v) * decay
        for (int d = 0; d < D; ++d) a[d] = 0.0;
        for (int n = 0; n < Np; ++n) {
          const double qn = q[n];
          double* rn = r.data() + static_cast<size_t>(n) * D;
          if (qn != 0.0)
            for (int d = 0; d < D; ++d) a[d] += qn * rn[d];
          for (int d = 0; d < D; ++d) rn[d] = (rn[d] + qn * c[d]) * decay;
        }
        layer_norm(a.data(), lna.data(), D);
        double* out = &xy_all[(static_cast<size_t>(t) * H + h) * N];
        for (int n = 0; n < N; ++n) {
          const float* w = encoder_v + (static_cast<size_t>(h) * N + n) * D;
          double s = 0.0;
          for (int d = 0; d < D; ++d) s += lna[d] * w[d];
          s -= relu_threshold;
          out[n] = (s > 0.0 ? s : 0.0) * xh[n];
        }
      }
      if (rho_out && l == L - 1)
        std::copy(r.begin(), r.end(), rho_out + static_cast<size_t>(h) * Np * D);
    };
    {
      std::vector<std::thread> pool;
      for (int h0 = 0; h0 < H; h0 += hw) {
        pool.clear();
        for (int h = h0; h < std::min(H, h0 + hw); ++h) pool.emplace_back(head_pass, h);
        for (auto& th : pool) th.join();
      }
    }
    auto token_pass = [&](int t0, int t1) {
      std::vector<double> mlp(D), tmp(D);
      for (int t = t0; t < t1; ++t) {
        const double* c = &cur[static_cast<size_t>(t) * D];
        const double* xy = &xy_all[static_cast<size_t>(t) * H * N];
        for (int d = 0; d < D; ++d) mlp[d] = 0.0;
        for (size_t k = 0; k < static_cast<size_t>(H) * N; ++k) {
          const double v = xy[k];
          if (v == 0.0) continue;
          const float* w = decoder + k * D;
          for (int d = 0; d < D; ++d) mlp[d] += v * w[d];
        }
        layer_norm(mlp.data(), tmp.data(), D);
        for (int d = 0; d < D; ++d) tmp[d] += c[d];
        layer_norm(tmp.data(), &nxt[static_cast<size_t>(t) * D], D);
      }
    };
    {
      const int parts = std::min(hw, T);
      std::vector<std::thread> pool;
      for (int p = 0; p < parts; ++p)
        pool.emplace_back(token_pass, static_cast<int>(static_cast<long long>(T) * p / parts),
                          static_cast<int>(static_cast<long long>(T) * (p + 1) / parts));
      for (auto& th : pool) th.join();
    }
    cur.swap(nxt);
  }
  for (int t = 0; t < T; ++t)
    for (int v = 0; v < V; ++v) {
      double s = 0.0;
      for (int d = 0; d < D; ++d) s += cur[static_cast<size_t>(t) * D + d] * lm_head[static_cast<size_t>(d) * V + v];
      logits[static_cast<size_t>(t) * V + v] = static_cast<float>(s);
    }
  return 0;
}

}  // extern "C"
