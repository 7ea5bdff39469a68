/* CPU oracle for the FaStar MLA layer.  TEST INFRASTRUCTURE ONLY: the checker for the CUDA
 * path and the timed host-CPU baseline.  See mla_oracle.h for the parity status.
 *
 * Every function names the reference lines it restates (paths are relative to the FaStar
 * source tree).  Deliberate differences from the NPU path, all far below the acceptance
 * tolerance: fp32 -> bf16 uses round-to-nearest-even where the reference truncates
 * (src/fst_engine.cpp:27); RoPE tables stay fp32 unless asked (the reference rounds them to
 * bf16, 1988-1989); the QK product is kept in fp32 (the NPU tile returns bf16); RMSNorm uses
 * the clean fp32 form of rms_cpu (89-91), not the AIE kernel's bf16 inverse-rms.
 */
#include "mla_oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include <sched.h>

namespace {

inline float bf16_rne(float x) {
  uint32_t b;
  std::memcpy(&b, &x, 4);
  if ((b & 0x7fffffffu) > 0x7f800000u) return x; /* NaN stays NaN */
  b += 0x7fffu + ((b >> 16) & 1u);
  b &= 0xffff0000u;
  float y;
  std::memcpy(&y, &b, 4);
  return y;
}

inline float bf16_trunc(float x) {
  uint32_t b;
  std::memcpy(&b, &x, 4);
  b &= 0xffff0000u;
  float y;
  std::memcpy(&y, &b, 4);
  return y;
}

inline float rnd(float x, int round_bf16) { return round_bf16 ? bf16_rne(x) : x; }

int available_cores() {
  cpu_set_t set;
  CPU_ZERO(&set);
  if (sched_getaffinity(0, sizeof(set), &set) == 0) {
    int n = CPU_COUNT(&set);
    if (n > 0) return n;
  }
  unsigned h = std::thread::hardware_concurrency();
  return h ? (int)h : 1;
}

int resolve_threads(int n) { return n > 0 ? n : available_cores(); }

/* Static block partition of [0, n) over worker threads. */
void parallel_for(int64_t n, int n_threads, const std::function<void(int64_t, int64_t)>& fn) {
  n_threads = (int)std::min<int64_t>(resolve_threads(n_threads), std::max<int64_t>(n, 1));
  if (n_threads <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> th;
  int64_t chunk = (n + n_threads - 1) / n_threads;
  for (int t = 0; t < n_threads; ++t) {
    int64_t a = t * chunk, b = std::min<int64_t>(n, a + chunk);
    if (a >= b) break;
    th.emplace_back([=, &fn] { fn(a, b); });
  }
  for (auto& t : th) t.join();
}

/* Work items [0, n) handed out one at a time from a shared counter: for items of uneven cost
 * (sequences of different lengths). */
void parallel_dynamic(int64_t n, int n_threads, const std::function<void(int64_t)>& fn) {
  n_threads = (int)std::min<int64_t>(resolve_threads(n_threads), std::max<int64_t>(n, 1));
  if (n_threads <= 1) {
    for (int64_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<int64_t> next{0};
  std::vector<std::thread> th;
  for (int t = 0; t < n_threads; ++t)
    th.emplace_back([&] {
      for (int64_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
    });
  for (auto& t : th) t.join();
}

/* Dot product with 16 fixed-order fp32 partial sums folded in double: deterministic,
 * vectorisable, and as accurate as the double-precision audits of the reference
 * (src/fst_engine.cpp:3375-3377) need it to be. */
inline float dot(const float* __restrict a, const float* __restrict b, int n) {
  float acc[16] = {0};
  int i = 0;
  for (; i + 16 <= n; i += 16)
    for (int j = 0; j < 16; ++j) acc[j] += a[i + j] * b[i + j];
  double s = 0;
  for (int j = 0; j < 16; ++j) s += acc[j];
  for (; i < n; ++i) s += (double)a[i] * b[i];
  return (float)s;
}

struct Dims {
  int H, hidden, q_lora, kv_lora, nope, rope, v_head, row, d_qk, d_v, q_head, low;
};

Dims dims_of(const FstOracleCfg* c) {
  Dims d;
  d.H = c->n_heads;
  d.hidden = c->hidden;
  d.q_lora = c->q_lora;
  d.kv_lora = c->kv_lora;
  d.rope = c->qk_rope;
  if (c->preset == FST_ORACLE_PRESET_BASELINE) {
    d.nope = c->qk_nope;
    d.v_head = c->v_head;
    d.row = c->kv_lora + c->qk_rope; /* [latent | k_pe] */
    d.d_qk = d.row;
    d.d_v = c->kv_lora;
    d.q_head = c->qk_nope + c->qk_rope;
    d.low = c->n_heads * c->v_head;
  } else {
    d.nope = c->kv_lora - c->qk_rope; /* 448 nope + 64 rope share the row */
    d.v_head = 0;
    d.row = c->kv_lora;
    d.d_qk = c->kv_lora;
    d.d_v = c->kv_lora;
    d.q_head = c->kv_lora;
    d.low = c->o_groups * c->o_lora;
  }
  return d;
}

}  // namespace

extern "C" {

int fst_oracle_row_width(const FstOracleCfg* c) { return dims_of(c).row; }
int fst_oracle_d_qk(const FstOracleCfg* c) { return dims_of(c).d_qk; }
int fst_oracle_d_v(const FstOracleCfg* c) { return dims_of(c).d_v; }
int fst_oracle_low_dim(const FstOracleCfg* c) { return dims_of(c).low; }
int fst_oracle_threads(const FstOracleCfg* c) { return resolve_threads(c->n_threads); }

float fst_oracle_bf16_round(float x) { return bf16_rne(x); }
float fst_oracle_bf16_trunc(float x) { return bf16_trunc(x); }
void fst_oracle_bf16_round_array(float* x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) x[i] = bf16_rne(x[i]);
}

/* rms_cpu, src/fst_engine.cpp:89-91: fp32 sum of squares, r = 1/sqrt(ss/d + eps),
 * y = x * r * w.  The per-head weightless form (3487-3495) is the w == NULL case. */
void fst_oracle_rmsnorm(const float* x, const float* w, float* y, int rows, int d, float eps,
                        int round_bf16) {
  for (int t = 0; t < rows; ++t) {
    const float* xi = x + (size_t)t * d;
    float* yo = y + (size_t)t * d;
    double ss = 0;
    for (int j = 0; j < d; ++j) ss += (double)xi[j] * xi[j];
    float r = 1.0f / std::sqrt((float)(ss / (double)d) + eps);
    for (int j = 0; j < d; ++j) yo[j] = rnd(xi[j] * r * (w ? w[j] : 1.0f), round_bf16);
  }
}

/* build_rope_lut, src/fst_engine.cpp:1970-2023.  Plain layers: theta(pair j) = pos *
 * theta_scale^j with theta_scale = base^(-2/rope_dim), accumulated by repeated fp32
 * multiplication exactly as there (1983-1991).  YaRN layers (1995-2022): base 160000,
 * freq_scale 1/16, n_ctx_orig 65536, beta_fast 32, beta_slow 1, ramp-mixed angle. */
void fst_oracle_rope_lut(float* lut, int pos, int rope_dim, float theta, int yarn, int inverse,
                         int round_lut_bf16) {
  const float sin_sign = inverse ? -1.0f : 1.0f;
  const float freq_base = yarn ? 160000.0f : theta;
  const float theta_scale = std::pow(freq_base, -2.0f / (float)rope_dim);
  float theta_extrap = (float)pos;
  if (!yarn) {
    for (int d = 0; d < rope_dim; d += 2) {
      float c = std::cos(theta_extrap), s = sin_sign * std::sin(theta_extrap);
      lut[d] = round_lut_bf16 ? bf16_trunc(c) : c;
      lut[d + 1] = round_lut_bf16 ? bf16_trunc(s) : s;
      theta_extrap *= theta_scale;
    }
    return;
  }
  const float freq_scale = 1.0f / 16.0f, ext_factor = 1.0f, n_ctx_orig = 65536.0f;
  const float beta_fast = 32.0f, beta_slow = 1.0f;
  auto corr_dim = [&](float beta) {
    return (float)rope_dim * std::log(n_ctx_orig / (beta * 2.0f * (float)M_PI)) /
           (2.0f * std::log(freq_base));
  };
  float corr0 = std::max(0.0f, std::floor(corr_dim(beta_fast)));
  float corr1 = std::min((float)(rope_dim - 1), std::ceil(corr_dim(beta_slow)));
  for (int d = 0; d < rope_dim; d += 2) {
    float y = ((float)(d / 2) - corr0) / std::max(0.001f, corr1 - corr0);
    float ramp_mix = (1.0f - std::min(1.0f, std::max(0.0f, y))) * ext_factor;
    float theta_interp = freq_scale * theta_extrap;
    float th = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
    float c = std::cos(th), s = sin_sign * std::sin(th);
    lut[d] = round_lut_bf16 ? bf16_trunc(c) : c;
    lut[d + 1] = round_lut_bf16 ? bf16_trunc(s) : s;
    theta_extrap *= theta_scale;
  }
}

/* ew_rope, kernels/fst_ew_unified_kernel.cc:200-217: (x0, x1) -> (x0 c - x1 s, x0 s + x1 c)
 * on interleaved pairs. */
void fst_oracle_rope_apply(float* x, int pos, int rope_dim, float theta, int yarn, int inverse,
                           int round_bf16) {
  std::vector<float> lut(rope_dim);
  fst_oracle_rope_lut(lut.data(), pos, rope_dim, theta, yarn, inverse, 0);
  for (int d = 0; d < rope_dim; d += 2) {
    float c = lut[d], s = lut[d + 1], x0 = x[d], x1 = x[d + 1];
    x[d] = rnd(x0 * c - x1 * s, round_bf16);
    x[d + 1] = rnd(x0 * s + x1 * c, round_bf16);
  }
}

/* npu_gemm_mla_vec semantics, src/fst_engine.cpp:465-575: C = A * B^T for the b_col_maj
 * kernels (weights in native [N,K]), C = A * B for the b_row_maj qksv kernel (480). */
void fst_oracle_gemm(const float* A, const float* B, float* C, int M, int N, int K, int b_kn,
                     int round_bf16, int n_threads) {
  if (!b_kn) {
    parallel_for(N, n_threads, [&](int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n)
        for (int m = 0; m < M; ++m)
          C[(size_t)m * N + n] = rnd(dot(A + (size_t)m * K, B + (size_t)n * K, K), round_bf16);
    });
  } else {
    parallel_for(M, n_threads, [&](int64_t m0, int64_t m1) {
      std::vector<double> acc(N);
      for (int64_t m = m0; m < m1; ++m) {
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int k = 0; k < K; ++k) {
          double a = A[(size_t)m * K + k];
          const float* b = B + (size_t)k * N;
          for (int n = 0; n < N; ++n) acc[n] += a * b[n];
        }
        for (int n = 0; n < N; ++n) C[(size_t)m * N + n] = rnd((float)acc[n], round_bf16);
      }
    });
  }
}

}  /* extern "C" */

namespace {

/* One (query token, head) row of QK -> softmax -> SV over rows [0, S) of `cache` and, when the
 * layer has a compressor, over the first n_cmp rows of `cmp` as further columns (3565-3586). */
void attention_row(const FstOracleCfg* c, const Dims& d, const float* q, const float* cache, int S,
                   bool has_sink, float sink, std::vector<float>& sc, std::vector<double>& acc, float* o,
                   const float* cmp = nullptr, int n_cmp = 0) {
  const float scale = c->softmax_scale;
  const int rb = c->round_bf16;
  const int Stot = S + n_cmp;
  if ((int)sc.size() < Stot) sc.resize(Stot);
  auto row_of = [&](int s) { return s < S ? cache + (size_t)s * d.row : cmp + (size_t)(s - S) * d.row; };
  float mx = has_sink ? sink : -INFINITY;
  for (int s = 0; s < Stot; ++s) {
    sc[s] = dot(q, row_of(s), d.d_qk) * scale;
    mx = std::max(mx, sc[s]);
  }
  if (Stot <= 0 && !has_sink) {
    for (int j = 0; j < d.d_v; ++j) o[j] = 0.0f;
    return;
  }
  float sum = has_sink ? std::exp(sink - mx) : 0.0f;
  for (int s = 0; s < Stot; ++s) sum += std::exp(sc[s] - mx);
  const float inv = 1.0f / (sum + 1e-12f);
  std::fill(acc.begin(), acc.end(), 0.0);
  for (int s = 0; s < Stot; ++s) {
    const float p = rnd(std::exp(sc[s] - mx) * inv, rb);
    const float* v = row_of(s);
    for (int j = 0; j < d.d_v; ++j) acc[j] += (double)p * v[j];
  }
  for (int j = 0; j < d.d_v; ++j) o[j] = rnd((float)acc[j], rb);
}

/* The 127 non-negative E4M3 values (3070-3083). */
const float* e4m3_grid() {
  static float g[127];
  static bool init = false;
  if (!init) {
    static const float exp_scale[16] = {0.0f, 0.015625f, 0.03125f, 0.0625f, 0.125f, 0.25f, 0.5f, 1.0f,
                                        2.0f, 4.0f,      8.0f,     16.0f,   32.0f,  64.0f, 128.0f, 256.0f};
    for (int i = 0; i < 127; ++i) {
      const int e = (i >> 3) & 15, m = i & 7;
      g[i] = e == 0 ? (float)m * 0.001953125f : (1.0f + (float)m * 0.125f) * exp_scale[e];
    }
    init = true;
  }
  return g;
}

}  // namespace

extern "C" {

/* QK -> softmax -> SV of src/fst_engine.cpp:3573-3683 for one sequence.
 * Softmax (3614-3666): v = score * scale; max starts at the sink logit; sum starts at
 * exp(sink - max); p = exp(v - max) / (sum + 1e-12), rounded to bf16 (3651-3652); masked
 * columns (s > pos0 + i when causal, 3626) contribute nothing.  Without a sink the sink
 * terms are dropped.  SV (3668-3683): out = sum_s p[s] * row_s[:d_v]. */
void fst_oracle_attention(const FstOracleCfg* c, const float* q_eff, const float* cache,
                          int kv_len, int n_q, int pos0, int causal, const float* sinks,
                          float* out) {
  const Dims d = dims_of(c);
  parallel_for((int64_t)n_q * d.H, c->n_threads, [&](int64_t r0, int64_t r1) {
    std::vector<float> sc(std::max(kv_len, 1));
    std::vector<double> acc(d.d_v);
    for (int64_t r = r0; r < r1; ++r) {
      const int i = (int)(r / d.H), hh = (int)(r % d.H);
      int S = kv_len;
      if (causal) S = std::min(S, pos0 + i + 1);
      const bool has_sink = c->use_sink && sinks;
      attention_row(c, d, q_eff + (size_t)r * d.d_qk, cache, S, has_sink, has_sink ? sinks[hh] : 0.0f, sc, acc,
                    out + (size_t)r * d.d_v);
    }
  });
}

void fst_oracle_attention_partial(const FstOracleCfg* c, const float* q_eff, const float* cache,
                                  int s0, int s1, int n_q, int pos0, int causal, float* m,
                                  float* l, float* o) {
  const Dims d = dims_of(c);
  const float scale = c->softmax_scale;
  parallel_for((int64_t)n_q * d.H, c->n_threads, [&](int64_t r0, int64_t r1) {
    std::vector<float> sc(std::max(s1 - s0, 1));
    std::vector<double> acc(d.d_v);
    for (int64_t r = r0; r < r1; ++r) {
      const int i = (int)(r / d.H);
      const float* q = q_eff + (size_t)r * d.d_qk;
      int e = s1;
      if (causal) e = std::min(e, pos0 + i + 1);
      float mx = -INFINITY;
      for (int s = s0; s < e; ++s) {
        sc[s - s0] = dot(q, cache + (size_t)s * d.row, d.d_qk) * scale;
        mx = std::max(mx, sc[s - s0]);
      }
      std::fill(acc.begin(), acc.end(), 0.0);
      double sum = 0;
      for (int s = s0; s < e; ++s) {
        const float p = std::exp(sc[s - s0] - mx);
        sum += p;
        const float* v = cache + (size_t)s * d.row;
        for (int j = 0; j < d.d_v; ++j) acc[j] += (double)p * v[j];
      }
      m[r] = mx;
      l[r] = (float)sum;
      for (int j = 0; j < d.d_v; ++j) o[(size_t)r * d.d_v + j] = (float)acc[j];
    }
  });
}

/* Split-KV has no counterpart in the reference (it attends to at most 128 rows in one
 * piece); the merge is the identity softmax(x) = sum_p e^{m_p - M} (l_p, o_p) /
 * sum_p e^{m_p - M} l_p, with the sink of 3623/3636 entering as one more part
 * (m = sink, l = 1, o = 0). */
void fst_oracle_merge_partials(const FstOracleCfg* c, const float* m, const float* l,
                               const float* o, int n_parts, int rows, const float* sinks,
                               float* out) {
  const Dims d = dims_of(c);
  const bool has_sink = c->use_sink && sinks;
  for (int r = 0; r < rows; ++r) {
    float M = has_sink ? sinks[r % d.H] : -INFINITY;
    for (int p = 0; p < n_parts; ++p) M = std::max(M, m[(size_t)p * rows + r]);
    double den = has_sink ? std::exp(sinks[r % d.H] - M) : 0.0;
    std::vector<double> acc(d.d_v, 0.0);
    for (int p = 0; p < n_parts; ++p) {
      const float mp = m[(size_t)p * rows + r];
      if (mp == -INFINITY) continue;
      const double w = std::exp(mp - M);
      den += w * l[(size_t)p * rows + r];
      const float* op = o + ((size_t)p * rows + r) * d.d_v;
      for (int j = 0; j < d.d_v; ++j) acc[j] += w * op[j];
    }
    for (int j = 0; j < d.d_v; ++j)
      out[(size_t)r * d.d_v + j] = rnd(den > 0 ? (float)(acc[j] / (den + 1e-12)) : 0.0f,
                                       c->round_bf16);
  }
}

/* process_mla, src/fst_engine.cpp:3320-3890, stage by stage, for B sequences in one call.  The
 * reference runs one sequence per call; here the rows of all sequences share every projection
 * (one product over T = sum q_lens rows, the weights read once), and the per-sequence stages
 * (RoPE position, cache push, attention) follow each row's own sequence.  h[T, hidden] holds the
 * sequences' rows back to back; trace buffers are sized for T rows. */
int fst_oracle_compressor_width(int ratio, int kv_lora) { return ratio == 4 ? 2 * kv_lora : (ratio > 0 ? kv_lora : 0); }
int fst_oracle_compressor_rows(int ratio) { return ratio == 4 ? 8 : ratio; }

float fst_oracle_e4m3_roundtrip(float v) {
  const float* g = e4m3_grid();
  const float sign = v < 0.0f ? -1.0f : 1.0f;
  const float ax = std::min(std::fabs(v), 448.0f);
  int lo = 0, hi = 126;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (g[mid] <= ax) lo = mid; else hi = mid - 1;
  }
  int best = lo;
  if (best < 126) {
    const float bd = std::fabs(ax - g[best]), nd = std::fabs(ax - g[best + 1]);
    if (nd < bd || (nd == bd && ((best + 1) & 1) == 0 && (best & 1) != 0)) ++best;
  }
  return sign * g[best];
}

/* compress_token, src/fst_engine.cpp:3171-3318.  The two projections are bf16 tile outputs there
 * (3189-3193); with round_bf16 they are rounded here too.  The compressed row is stored as bf16
 * (3268-3271; the reference truncates, this build rounds to nearest like everywhere else -- the
 * nope part is exactly representable either way, only the 64 tail values can differ by one step). */
int fst_oracle_compress_token(const FstOracleCfg* c, const FstOracleCompressorW* w, FstOracleCompressorState* st,
                              const float* hidden_normed, int pos) {
  const Dims d = dims_of(c);
  const int ratio = w->ratio, hd = d.kv_lora;
  if (ratio <= 0) return 0;
  const int width = fst_oracle_compressor_width(ratio, hd);
  const int pos_mod = pos % ratio;
  const int row = ratio == 4 ? ratio + pos_mod : pos_mod;
  const bool should = ((pos + 1) % ratio) == 0;
  std::vector<float> kv_cur(width), sc_cur(width);
  for (int j = 0; j < width; ++j) {
    kv_cur[j] = rnd(dot(hidden_normed, w->wkv + (size_t)j * d.hidden, d.hidden), c->round_bf16);
    sc_cur[j] = rnd(dot(hidden_normed, w->wgate + (size_t)j * d.hidden, d.hidden), c->round_bf16) +
                w->ape[(size_t)pos_mod * width + j]; /* APE add, 3197-3198 */
  }
  std::memcpy(st->state_kv + (size_t)row * width, kv_cur.data(), width * sizeof(float));
  std::memcpy(st->state_sc + (size_t)row * width, sc_cur.data(), width * sizeof(float));
  if (!should) return 0;
  if (st->n_comp >= st->cap) return -1;

  /* per-dim softmax pool over the window rows, two lanes for ratio 4 (3206-3242) */
  std::vector<float> pooled(hd, 0.0f);
  for (int j = 0; j < hd; ++j) {
    float mx = -1e30f;
    for (int r = 0; r < ratio; ++r) {
      mx = std::max(mx, st->state_sc[(size_t)r * width + j]);
      if (ratio == 4) mx = std::max(mx, st->state_sc[(size_t)(ratio + r) * width + hd + j]);
    }
    if (mx <= -0.5e30f) continue;
    float denom = 0.0f, sum = 0.0f;
    for (int r = 0; r < ratio; ++r) {
      const float wp = std::exp(st->state_sc[(size_t)r * width + j] - mx);
      if (ratio == 4) {
        const float wc = std::exp(st->state_sc[(size_t)(ratio + r) * width + hd + j] - mx);
        denom += wp + wc;
        sum += wp * st->state_kv[(size_t)r * width + j];
        sum += wc * st->state_kv[(size_t)(ratio + r) * width + hd + j];
      } else {
        denom += wp;
        sum += wp * st->state_kv[(size_t)r * width + j];
      }
    }
    pooled[j] = denom > 0.0f ? sum / denom : 0.0f;
  }
  /* RMS norm with the compressor's weight (3244-3250) */
  double ss = 0;
  for (int i = 0; i < hd; ++i) ss += (double)pooled[i] * pooled[i];
  const float rms = 1.0f / std::sqrt((float)(ss / (double)hd) + 1e-6f);
  std::vector<float> out(hd);
  for (int i = 0; i < hd; ++i) out[i] = pooled[i] * rms * w->norm[i];
  /* RoPE on the tail at comp_pos = pos + 1 - ratio (3252-3254, rope_tail_yarn 3108-3153) */
  fst_oracle_rope_apply(out.data() + hd - d.rope, pos + 1 - ratio, d.rope, c->rope_theta, c->rope_yarn, 0, 0);
  /* E4M3 round trip of the nope part in 64-blocks (3256-3267) */
  for (int off = 0; off < hd - d.rope; off += 64) {
    float amax = 0.0f;
    for (int i = 0; i < 64; ++i) amax = std::max(amax, std::fabs(out[off + i]));
    if (amax < 1.0e-4f) amax = 1.0e-4f;
    const float scale = std::ldexp(1.0f, (int)std::ceil(std::log2(amax / 448.0f)));
    for (int i = 0; i < 64; ++i) {
      float v = out[off + i] / scale;
      v = std::min(448.0f, std::max(-448.0f, v));
      out[off + i] = fst_oracle_e4m3_roundtrip(v) * scale;
    }
  }
  for (int i = 0; i < hd; ++i) st->cache[(size_t)st->n_comp * hd + i] = bf16_rne(out[i]);
  st->n_comp++;
  /* window rotation, ratio 4 only (3302-3317): both lanes become the window just processed */
  if (ratio == 4) {
    for (int r = 0; r < ratio; ++r) {
      std::memcpy(st->state_kv + (size_t)r * width, st->state_kv + (size_t)(ratio + r) * width, width * sizeof(float));
      std::memcpy(st->state_sc + (size_t)r * width, st->state_sc + (size_t)(ratio + r) * width, width * sizeof(float));
    }
  }
  return 1;
}

int fst_oracle_mla_forward_batch(const FstOracleCfg* c, const FstOracleWeights* w, const float* h, int B,
                                 const int32_t* q_lens, const int32_t* pos0, int causal, float* const* caches,
                                 const int32_t* caps, float* out, FstOracleTrace* trace) {
  return fst_oracle_mla_forward_batch_cmp(c, w, nullptr, nullptr, h, B, q_lens, pos0, causal, caches, caps, out, trace);
}

int fst_oracle_mla_forward_batch_cmp(const FstOracleCfg* c, const FstOracleWeights* w,
                                     const FstOracleCompressorW* cw, FstOracleCompressorState* states,
                                     const float* h, int B, const int32_t* q_lens, const int32_t* pos0, int causal,
                                     float* const* caches, const int32_t* caps, float* out, FstOracleTrace* trace) {
  const Dims d = dims_of(c);
  const int rb = c->round_bf16, nt = c->n_threads;
  if (B < 0) return -1;
  std::vector<int> seq_of, pos_of, tok0(B + 1, 0);
  for (int b = 0; b < B; ++b) {
    if (pos0[b] < 0 || q_lens[b] < 0 || pos0[b] + q_lens[b] > caps[b]) return -1; /* assert at 3327 */
    for (int i = 0; i < q_lens[b]; ++i) {
      seq_of.push_back(b);
      pos_of.push_back(pos0[b] + i);
    }
    tok0[b + 1] = (int)seq_of.size();
  }
  const int T = (int)seq_of.size();
  if (T == 0) return 0;
  const bool v4 = c->preset == FST_ORACLE_PRESET_FASTAR_V4;

  /* attn_norm of process_layer (2687-2688), when its weight is given: an = rmsnorm(h) * w. */
  std::vector<float> an;
  if (w->attn_norm) {
    an.resize((size_t)T * d.hidden);
    fst_oracle_rmsnorm(h, w->attn_norm, an.data(), T, d.hidden, c->rms_eps, rb);
    h = an.data();
  }

  /* q compress (3362-3364) + q_norm (3385-3389). */
  std::vector<float> qc((size_t)T * d.q_lora);
  fst_oracle_gemm(h, w->wq_a, qc.data(), T, d.q_lora, d.hidden, 0, rb, nt);
  if (w->q_norm) fst_oracle_rmsnorm(qc.data(), w->q_norm, qc.data(), T, d.q_lora, c->rms_eps, rb);

  /* kv compress (3366-3368) + kv_norm on the kv_lora latent (3390-3394). BASELINE: the
   * projection has kv_lora + rope outputs and the trailing k_pe is not normed. */
  std::vector<float> kv((size_t)T * d.row);
  fst_oracle_gemm(h, w->wkv_a, kv.data(), T, d.row, d.hidden, 0, rb, nt);
  for (int m = 0; m < T; ++m) {
    float* r = kv.data() + (size_t)m * d.row;
    if (w->kv_norm) fst_oracle_rmsnorm(r, w->kv_norm, r, 1, d.kv_lora, c->rms_eps, rb);
    /* RoPE on the key's rope dims (3504-3517): V4 row tail, BASELINE the separate k_pe. */
    fst_oracle_rope_apply(r + d.row - d.rope, pos_of[m], d.rope, c->rope_theta, c->rope_yarn, 0, rb);
  }
  if (trace && trace->qc) std::memcpy(trace->qc, qc.data(), qc.size() * sizeof(float));
  if (trace && trace->kv) std::memcpy(trace->kv, kv.data(), kv.size() * sizeof(float));

  /* q expand (3409-3473). */
  const int qn = d.H * d.q_head;
  std::vector<float> q_full((size_t)T * qn);
  fst_oracle_gemm(qc.data(), w->wq_b, q_full.data(), T, qn, d.q_lora, 0, rb, nt);

  std::vector<float> q_eff((size_t)T * d.H * d.d_qk);
  if (v4) {
    /* per-head weightless RMSNorm (3487-3495), then RoPE on every head's tail (3503). */
    parallel_for((int64_t)T * d.H, nt, [&](int64_t r0, int64_t r1) {
      for (int64_t r = r0; r < r1; ++r) {
        float* qh = q_full.data() + (size_t)r * d.q_head;
        /* the draft layer has no head norm and rotates head 0 only (4950-4983) */
        if (!c->draft_form) fst_oracle_rmsnorm(qh, nullptr, qh, 1, d.q_head, c->rms_eps, rb);
        if (!c->draft_form || r % d.H == 0)
          fst_oracle_rope_apply(qh + d.nope, pos_of[r / d.H], d.rope, c->rope_theta, c->rope_yarn, 0, rb);
        std::memcpy(q_eff.data() + (size_t)r * d.d_qk, qh, d.q_head * sizeof(float));
      }
    });
  } else {
    /* BASELINE: rotate q_pe, absorb q_nope through W_UK (rows [h*(nope+v), +nope) of
     * wkv_b, each [kv_lora]): q_lat[c] = sum_n q_nope[n] * W_UK[h][n, c]. */
    parallel_for((int64_t)T * d.H, nt, [&](int64_t r0, int64_t r1) {
      std::vector<double> acc(d.kv_lora);
      for (int64_t r = r0; r < r1; ++r) {
        const int hh = (int)(r % d.H);
        float* qh = q_full.data() + (size_t)r * d.q_head;
        fst_oracle_rope_apply(qh + d.nope, pos_of[r / d.H], d.rope, c->rope_theta, c->rope_yarn, 0, rb);
        const float* wuk = w->wkv_b + (size_t)hh * (d.nope + d.v_head) * d.kv_lora;
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int n = 0; n < d.nope; ++n) {
          const double a = qh[n];
          const float* wr = wuk + (size_t)n * d.kv_lora;
          for (int j = 0; j < d.kv_lora; ++j) acc[j] += a * wr[j];
        }
        float* qe = q_eff.data() + (size_t)r * d.d_qk;
        for (int j = 0; j < d.kv_lora; ++j) qe[j] = rnd((float)acc[j], rb);
        std::memcpy(qe + d.kv_lora, qh + d.nope, d.rope * sizeof(float));
      }
    });
  }
  if (trace && trace->q_eff) std::memcpy(trace->q_eff, q_eff.data(), q_eff.size() * sizeof(float));

  /* cache push (3534-3544): rows pos0 .. pos0+M-1 of every sequence. */
  for (int b = 0; b < B; ++b)
    if (q_lens[b] > 0)
      std::memcpy(caches[b] + (size_t)pos0[b] * d.row, kv.data() + (size_t)tok0[b] * d.row,
                  (size_t)q_lens[b] * d.row * sizeof(float));

  /* KV compressor (3545-3568): the new rows, in order, after the push and before the attention. */
  const bool has_cmp = cw && cw->ratio > 0 && states;
  if (has_cmp)
    for (int t = 0; t < T; ++t)
      if (fst_oracle_compress_token(c, cw, &states[seq_of[t]], h + (size_t)t * d.hidden, pos_of[t]) < 0) return -1;

  /* QK, softmax, SV (3573-3683): a row (token, head) attends to S = pos0 + M rows of its own
   * sequence, minus the rows the causal mask drops (3626). */
  std::vector<float> o_lat((size_t)T * d.H * d.d_v);
  {
    const bool has_sink = c->use_sink && w->attn_sinks;
    parallel_dynamic((int64_t)T * d.H, nt, [&](int64_t r) {
      thread_local std::vector<float> sc;
      thread_local std::vector<double> acc;
      if ((int)acc.size() != d.d_v) acc.assign(d.d_v, 0.0);
      const int t = (int)(r / d.H), hh = (int)(r % d.H), b = seq_of[t];
      int S = pos0[b] + q_lens[b];
      if (causal) S = std::min(S, pos_of[t] + 1);
      /* compressed column k was emitted at position (k + 1) * ratio - 1: visible to every row in
       * decode, to rows at or after that position when causal (3630-3635) */
      int n_cmp = 0;
      if (has_cmp) {
        n_cmp = states[b].n_comp;
        if (causal) n_cmp = std::min(n_cmp, (pos_of[t] + 1) / cw->ratio);
      }
      const int lo = c->window > 0 ? std::max(0, S - c->window) : 0;
      attention_row(c, d, q_eff.data() + (size_t)r * d.d_qk, caches[b] + (size_t)lo * d.row, S - lo, has_sink,
                    has_sink ? w->attn_sinks[hh] : 0.0f, sc, acc, o_lat.data() + (size_t)r * d.d_v,
                    has_cmp ? states[b].cache : nullptr, n_cmp);
    });
  }

  /* V4: inverse RoPE on every head's output tail (3716). */
  if (v4)
    for (int r = 0; r < T * d.H; ++r)
      if (!c->draft_form || r % d.H == 0) /* the draft layer: head 0 only (5077-5093) */
        fst_oracle_rope_apply(o_lat.data() + (size_t)r * d.d_v + d.nope, pos_of[r / d.H], d.rope,
                              c->rope_theta, c->rope_yarn, 1, rb);
  if (trace && trace->o_lat) std::memcpy(trace->o_lat, o_lat.data(), o_lat.size() * sizeof(float));

  /* O-proj a. V4 (3736-3839): low[:, g*o_lora:(g+1)*o_lora] = heads[:, g*gk:(g+1)*gk] *
   * wo_a[g*o_lora:(g+1)*o_lora, :]^T with gk = H*512/o_groups.  BASELINE: the per-head
   * W_UV (rows [h*(nope+v)+nope, +v) of wkv_b): low[h*v + j] = sum_c W_UV[h][j,c] o_lat[h][c]. */
  std::vector<float> low((size_t)T * d.low);
  if (v4) {
    const int gk = d.H * d.d_v / c->o_groups;
    parallel_for((int64_t)c->o_groups * c->o_lora, nt, [&](int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n) {
        const int g = (int)(n / c->o_lora);
        for (int m = 0; m < T; ++m)
          low[(size_t)m * d.low + n] = rnd(
              dot(o_lat.data() + (size_t)m * d.H * d.d_v + (size_t)g * gk, w->wo_a + (size_t)n * gk, gk), rb);
      }
    });
  } else {
    parallel_for((int64_t)d.H * d.v_head, nt, [&](int64_t n0, int64_t n1) {
      for (int64_t n = n0; n < n1; ++n) {
        const int hh = (int)(n / d.v_head), j = (int)(n % d.v_head);
        const float* wuv = w->wkv_b + ((size_t)hh * (d.nope + d.v_head) + d.nope + j) * d.kv_lora;
        for (int m = 0; m < T; ++m)
          low[(size_t)m * d.low + n] =
              rnd(dot(o_lat.data() + ((size_t)m * d.H + hh) * d.d_v, wuv, d.d_v), rb);
      }
    });
  }
  if (trace && trace->low) std::memcpy(trace->low, low.data(), low.size() * sizeof(float));

  /* O-proj b (3853-3868): attn_out = low * wo_b^T, written back over h by the caller (3889). */
  fst_oracle_gemm(low.data(), w->wo_b, out, T, d.hidden, d.low, 0, rb, nt);
  return 0;
}

/* The reference's own call shape: one sequence, M new rows at pos0 .. pos0+M-1. */
int fst_oracle_mla_forward(const FstOracleCfg* c, const FstOracleWeights* w, const float* h, int M,
                           int pos0, int causal, float* cache, int cap, float* out,
                           FstOracleTrace* trace) {
  const int32_t q = M, p = pos0, cp = cap;
  float* caches[1] = {cache};
  return fst_oracle_mla_forward_batch(c, w, h, 1, &q, &p, causal, caches, &cp, out, trace);
}

/* ---- paged-cache bookkeeping twin ------------------------------------------------------
 * The reference cache is one flat [max_seq, 512] buffer per layer addressed by seq_pos_
 * (include/fst_engine.h:108-113, src/fst_engine.cpp:1469-1474, 3536).  The paged form maps
 * token t of a sequence to (table[t / page_tokens], t % page_tokens); pages come from a
 * LIFO free list that initially hands out 0, 1, 2, ... */
struct FstOraclePager {
  int n_pages, page_tokens, max_seqs;
  std::vector<int32_t> free_pages; /* stack: back() is handed out next */
  std::vector<int32_t> free_seqs;
  std::vector<std::vector<int32_t>> tables;
  std::vector<int> lens;
  std::vector<char> live;
};

FstOraclePager* fst_oracle_pager_create(int n_pages, int page_tokens, int max_seqs) {
  if (n_pages < 0 || page_tokens <= 0 || max_seqs <= 0) return nullptr;
  auto* p = new FstOraclePager;
  p->n_pages = n_pages;
  p->page_tokens = page_tokens;
  p->max_seqs = max_seqs;
  for (int i = n_pages - 1; i >= 0; --i) p->free_pages.push_back(i);
  for (int i = max_seqs - 1; i >= 0; --i) p->free_seqs.push_back(i);
  p->tables.resize(max_seqs);
  p->lens.assign(max_seqs, 0);
  p->live.assign(max_seqs, 0);
  return p;
}
void fst_oracle_pager_destroy(FstOraclePager* p) { delete p; }

int fst_oracle_pager_seq_alloc(FstOraclePager* p) {
  if (p->free_seqs.empty()) return -1;
  int s = p->free_seqs.back();
  p->free_seqs.pop_back();
  p->live[s] = 1;
  p->lens[s] = 0;
  p->tables[s].clear();
  return s;
}

int fst_oracle_pager_truncate(FstOraclePager* p, int seq, int n_tokens) {
  if (seq < 0 || seq >= p->max_seqs || !p->live[seq] || n_tokens < 0 || n_tokens > p->lens[seq])
    return -1;
  size_t keep = ((size_t)n_tokens + p->page_tokens - 1) / p->page_tokens;
  auto& t = p->tables[seq];
  while (t.size() > keep) {
    p->free_pages.push_back(t.back());
    t.pop_back();
  }
  p->lens[seq] = n_tokens;
  return 0;
}

int fst_oracle_pager_seq_free(FstOraclePager* p, int seq) {
  if (fst_oracle_pager_truncate(p, seq, 0) != 0) return -1;
  p->live[seq] = 0;
  p->free_seqs.push_back(seq);
  return 0;
}

int fst_oracle_pager_reserve(FstOraclePager* p, int seq, int n_tokens) {
  if (seq < 0 || seq >= p->max_seqs || !p->live[seq] || n_tokens < 0) return -1;
  size_t need = ((size_t)n_tokens + p->page_tokens - 1) / p->page_tokens;
  auto& t = p->tables[seq];
  if (need > t.size() && need - t.size() > p->free_pages.size()) return -2;
  while (t.size() < need) {
    t.push_back(p->free_pages.back());
    p->free_pages.pop_back();
  }
  p->lens[seq] = std::max(p->lens[seq], n_tokens);
  return 0;
}

int fst_oracle_pager_table(const FstOraclePager* p, int seq, int32_t* out, int cap) {
  if (seq < 0 || seq >= p->max_seqs || !p->live[seq]) return -1;
  const auto& t = p->tables[seq];
  for (size_t i = 0; i < t.size() && (int)i < cap; ++i) out[i] = t[i];
  return (int)t.size();
}

int fst_oracle_pager_free_pages(const FstOraclePager* p) { return (int)p->free_pages.size(); }

}  /* extern "C" */
