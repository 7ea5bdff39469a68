// CUDA-core kernels of the MLA path: the small fused stages (norms, RoPE, cache append,
// log-sum-exp merge) and shape-agnostic GEMM / attention kernels used where the tcgen05
// kernels do not apply (odd shapes, the [K,N] absorb operand) and for bisecting.
#include "kernels.cuh"
#include "tc_common.cuh"

namespace fst {

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// ---- GEMM, B in [N, K] (npu_gemm_mla_vec b_col_maj, reference src/fst_engine.cpp:477-484) ----
// A warp owns a 8 x 4 output tile; its lanes split K in 16-byte pieces.
template <bool VEC>
__global__ void __launch_bounds__(128) k_gemm_nk(GemmArgs g) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bf16* A = g.A + (long long)blockIdx.z * g.a_bs;
  const bf16* B = g.B + (long long)blockIdx.z * g.b_bs;
  bf16* C = g.C + (long long)blockIdx.z * g.c_bs;
  const int n0 = (blockIdx.x * 4 + warp) * 4, m0 = blockIdx.y * 8;
  if (n0 >= g.N) return;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  if (VEC) {
    for (int k = lane * 8; k < g.K; k += 256) {
      float b[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = min(n0 + j, g.N - 1);
        unpack8(*reinterpret_cast<const uint4*>(B + (long long)n * g.ldb + k), b[j]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = min(m0 + i, g.M - 1);
        float a[8];
        unpack8(*reinterpret_cast<const uint4*>(A + (long long)m * g.lda + k), a);
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][j] = fmaf(a[e], b[j][e], acc[i][j]);
      }
    }
  } else {
    for (int k = lane; k < g.K; k += 32) {
      float b[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = bf2f(B[(long long)min(n0 + j, g.N - 1) * g.ldb + k]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float a = bf2f(A[(long long)min(m0 + i, g.M - 1) * g.lda + k]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a, b[j], acc[i][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float v = warp_sum(acc[i][j]);
      if (lane == 0 && m0 + i < g.M && n0 + j < g.N) C[(long long)(m0 + i) * g.ldc + n0 + j] = f2bf(v);
    }
}

// ---- GEMM, B in [K, N] (the b_row_maj operand, reference src/fst_engine.cpp:480) ----
__global__ void __launch_bounds__(128) k_gemm_kn(GemmArgs g) {
  pdl_launch();
  pdl_wait();
  const bf16* A = g.A + (long long)blockIdx.z * g.a_bs;
  const bf16* B = g.B + (long long)blockIdx.z * g.b_bs;
  bf16* C = g.C + (long long)blockIdx.z * g.c_bs;
  const int n = blockIdx.x * 128 + threadIdx.x;
  const int m0 = blockIdx.y * 8;
  if (n >= g.N) return;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int k = 0; k < g.K; ++k) {
    const float b = bf2f(B[(long long)k * g.ldb + n]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      acc[i] = fmaf(bf2f(A[(long long)min(m0 + i, g.M - 1) * g.lda + k]), b, acc[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (m0 + i < g.M) C[(long long)(m0 + i) * g.ldc + n] = f2bf(acc[i]);
}

void launch_gemm_simt(const GemmArgs& g, cudaStream_t st) {
  if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return;
  if (g.b_kn) {
    dim3 grid((g.N + 127) / 128, (g.M + 7) / 8, g.batch);
    launch_pdl(k_gemm_kn, grid, dim3(128), 0, st, 1, g);
    return;
  }
  dim3 grid((g.N + 15) / 16, (g.M + 7) / 8, g.batch);
  const bool vec = g.K % 8 == 0 && g.lda % 8 == 0 && g.ldb % 8 == 0 && g.a_bs % 8 == 0 &&
                   g.b_bs % 8 == 0 && (reinterpret_cast<uintptr_t>(g.A) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(g.B) & 15) == 0;
  if (vec)
    launch_pdl(k_gemm_nk<true>, grid, dim3(128), 0, st, 1, g);
  else
    launch_pdl(k_gemm_nk<false>, grid, dim3(128), 0, st, 1, g);
}

// ---- attn_norm ---------------------------------------------------------------------------------
// One block per row; the row is loaded once (up to 32 elements per thread) and reduced once.
__global__ void __launch_bounds__(256) k_rmsnorm_rows(const bf16* x, const bf16* w, bf16* y, int dim, float eps) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x, tid = threadIdx.x;
  const bf16* in = x + (long long)t * dim;
  float v[32], g[32];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int j = tid + i * 256;
    v[i] = j < dim ? bf2f(in[j]) : 0.0f;
    g[i] = j < dim ? bf2f(w[j]) : 0.0f;
    ss += v[i] * v[i];
  }
  ss = block_sum(ss, scratch);
  const float r = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int j = tid + i * 256;
    if (j < dim) y[(long long)t * dim + j] = f2bf(v[i] * r * g[i]);
  }
}

void launch_rmsnorm_rows(const bf16* x, const bf16* w, bf16* y, int T, int dim, float eps, cudaStream_t st) {
  if (T <= 0) return;
  launch_pdl(k_rmsnorm_rows, dim3(T), dim3(256), 0, st, 1, x, w, y, dim, eps);
}

// ---- q_norm / kv_norm / key RoPE / cache append -------------------------------------------
// Reference src/fst_engine.cpp:3385-3394 (norms), 3504-3517 (RoPE on the key), 3534-3544
// (cache push).  One block per new token.  RMSNorm follows rms_cpu (89-91).
// Every global load of a block (its row of the compressed activations, the norm weights, the RoPE
// table, the destination) is issued before anything is reduced, and the two sums of squares
// share one exchange: the kernel is one memory round trip and one block reduction long.
__global__ void __launch_bounds__(256) k_norm_append(NormAppendArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float s_row[];  // [row]
  __shared__ float scratch[2][32];
  constexpr int QMAX = 8, KMAX = 4;  // q_lora <= 2048, row <= 1024 (checked by the launcher)
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const bf16* in = a.cmp + (long long)t * (a.q_lora + a.row);
  const bf16* kin = in + a.q_lora;
  float xq[QMAX], wq[QMAX], xk[KMAX], wk[KMAX];
#pragma unroll
  for (int i = 0; i < QMAX; ++i) {
    const int j = tid + i * 256;
    xq[i] = j < a.q_lora ? bf2f(in[j]) : 0.0f;
    wq[i] = (j < a.q_lora && a.q_norm) ? bf2f(a.q_norm[j]) : 1.0f;
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int j = tid + i * 256;
    xk[i] = j < a.row ? bf2f(kin[j]) : 0.0f;
    wk[i] = (j < a.kv_lora && a.kv_norm) ? bf2f(a.kv_norm[j]) : 1.0f;
  }
  const float* lut = a.lut + (long long)t * a.rope;
  float lc = 0.0f, ls = 0.0f;
  if (tid < a.rope / 2) {
    lc = lut[2 * tid];
    ls = lut[2 * tid + 1];
  }
  const long long dst = a.dst_row[t];
  // sums of squares: q over q_lora, kv over the kv_lora latent (trailing dims pass through)
  float sq = 0.0f, sk = 0.0f;
#pragma unroll
  for (int i = 0; i < QMAX; ++i) sq += xq[i] * xq[i];  // absent elements are 0
#pragma unroll
  for (int i = 0; i < KMAX; ++i)
    if (tid + i * 256 < a.kv_lora) sk += xk[i] * xk[i];
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) {
    scratch[0][wid] = sq;
    scratch[1][wid] = sk;
  }
  __syncthreads();
  sq = warp_sum(lane < nw ? scratch[0][lane] : 0.0f);
  sk = warp_sum(lane < nw ? scratch[1][lane] : 0.0f);
  const float rq = 1.0f / sqrtf(sq / (float)a.q_lora + a.eps);
  const float rk = 1.0f / sqrtf(sk / (float)a.kv_lora + a.eps);
#pragma unroll
  for (int i = 0; i < QMAX; ++i) {
    const int j = tid + i * 256;
    if (j < a.q_lora) a.qc[(long long)t * a.q_lora + j] = f2bf(a.q_norm ? xq[i] * rq * wq[i] : xq[i]);
  }
#pragma unroll
  for (int i = 0; i < KMAX; ++i) {
    const int j = tid + i * 256;
    if (j < a.row) s_row[j] = (j < a.kv_lora && a.kv_norm) ? rbf(xk[i] * rk * wk[i]) : xk[i];
  }
  __syncthreads();
  // RoPE on the last `rope` dims of the row, interleaved pairs (ew_rope,
  // reference kernels/fst_ew_unified_kernel.cc:200-217)
  if (tid < a.rope / 2) {
    const int j = a.row - a.rope + 2 * tid;
    const float x0 = s_row[j], x1 = s_row[j + 1];
    s_row[j] = x0 * lc - x1 * ls;
    s_row[j + 1] = x0 * ls + x1 * lc;
  }
  __syncthreads();
  for (int j = tid; j < a.row; j += blockDim.x) {
    const bf16 v = f2bf(s_row[j]);
    a.kv_new[(long long)t * a.row + j] = v;
    if (dst >= 0) a.pool[dst + j] = v;
  }
}

void launch_norm_append(const NormAppendArgs& a, cudaStream_t st) {
  if (a.T <= 0) return;
  launch_pdl(k_norm_append, dim3(a.T), dim3(256), a.row * sizeof(float), st, 1, a);
}

// ---- query preparation -----------------------------------------------------------------------
// BASELINE: rotate the rope dims of every head of q_full into q_eff[:, kv_lora:]
// (rope_qpe_all_heads, reference src/fst_engine.cpp:2025-2058; the absorb GEMM fills the rest).
// V4: per-head weightless RMSNorm (3487-3495), then the tail rotation (3503).
__global__ void __launch_bounds__(128) k_q_prep(QPrepArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ float s_q[1024];
  const int r = blockIdx.x, t = r / a.H;
  const bf16* in = a.q_full + (long long)r * a.q_head;
  bf16* out = a.q_eff + (long long)r * a.d_qk;
  const float* lut = a.lut + (long long)t * a.rope;
  if (a.v4) {
    float sc = 1.0f;
    if (a.head_norm) {
      float ss = 0.0f;
      for (int j = threadIdx.x; j < a.q_head; j += blockDim.x) {
        const float x = bf2f(in[j]);
        ss += x * x;
      }
      ss = block_sum(ss, scratch);
      sc = 1.0f / sqrtf(ss / (float)a.q_head + a.eps);
    }
    for (int j = threadIdx.x; j < a.q_head; j += blockDim.x) s_q[j] = rbf(bf2f(in[j]) * sc);
    __syncthreads();
    for (int p = threadIdx.x; p < a.rope / 2 && r % a.H < a.rope_heads; p += blockDim.x) {
      const int j = a.nope + 2 * p;
      const float c = lut[2 * p], s = lut[2 * p + 1], x0 = s_q[j], x1 = s_q[j + 1];
      s_q[j] = x0 * c - x1 * s;
      s_q[j + 1] = x0 * s + x1 * c;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < a.q_head; j += blockDim.x) out[j] = f2bf(s_q[j]);
  } else {
    for (int p = threadIdx.x; p < a.rope / 2; p += blockDim.x) {
      const float c = lut[2 * p], s = lut[2 * p + 1];
      const float x0 = bf2f(in[a.nope + 2 * p]), x1 = bf2f(in[a.nope + 2 * p + 1]);
      out[a.d_qk - a.rope + 2 * p] = f2bf(x0 * c - x1 * s);
      out[a.d_qk - a.rope + 2 * p + 1] = f2bf(x0 * s + x1 * c);
    }
  }
}

// BASELINE only: one block per token rotates the rope pairs of all its heads (a pair per thread
// and step) -- a handful of fat blocks instead of T * H blocks of 32 busy threads.
__global__ void __launch_bounds__(256) k_q_rope_token(QPrepArgs a) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x, half = a.rope / 2;
  const float* lut = a.lut + (long long)t * a.rope;
  for (int i = threadIdx.x; i < a.H * half; i += blockDim.x) {
    const int h = i / half, p = i % half;
    const bf16* in = a.q_full + ((long long)t * a.H + h) * a.q_head + a.nope + 2 * p;
    bf16* out = a.q_eff + ((long long)t * a.H + h) * a.d_qk + a.d_qk - a.rope + 2 * p;
    const float c = lut[2 * p], s = lut[2 * p + 1];
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(in);
    const float x0 = __low2float(x), x1 = __high2float(x);
    *reinterpret_cast<__nv_bfloat162*>(out) = __floats2bfloat162_rn(x0 * c - x1 * s, x0 * s + x1 * c);
  }
}

// V4: a warp per (token, head) row, eight rows per block: the row (q_head <= 1024 values) stays in
// registers, 16 bytes per lane and pass; one shuffle reduction instead of two block barriers and a
// shared-memory round trip per row.  Same order of operations per element as k_q_prep.
__global__ void __launch_bounds__(256) k_q_prep_v4_rows(QPrepArgs a) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * 8 + warp;
  if (r >= (long long)a.T * a.H) return;
  const int t = (int)(r / a.H), h = (int)(r % a.H);
  const uint4* in = reinterpret_cast<const uint4*>(a.q_full + r * a.q_head);
  uint4* out = reinterpret_cast<uint4*>(a.q_eff + r * a.d_qk);
  const float* lut = a.lut + (long long)t * a.rope;
  const int n_u = a.q_head / 8;
  float x[4][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = lane + 32 * i;
    if (u < n_u) {
      const uint4 v = in[u];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
        x[i][2 * e] = __low2float(b);
        x[i][2 * e + 1] = __high2float(b);
        ss += x[i][2 * e] * x[i][2 * e] + x[i][2 * e + 1] * x[i][2 * e + 1];
      }
    }
  }
  ss = warp_sum(ss);
  const float sc = a.head_norm ? 1.0f / sqrtf(ss / (float)a.q_head + a.eps) : 1.0f;
  const bool rot = h < a.rope_heads;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int u = lane + 32 * i;
    if (u < n_u) {
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) y[e] = rbf(x[i][e] * sc);
      const int j0 = 8 * u - a.nope;  // first rope dim of this unit, if not negative
      if (rot && j0 >= 0) {
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float c = lut[j0 + e], sn = lut[j0 + e + 1], x0 = y[e], x1 = y[e + 1];
          y[e] = x0 * c - x1 * sn;
          y[e + 1] = x0 * sn + x1 * c;
        }
      }
      uint32_t pk[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(y[2 * e], y[2 * e + 1]);
        pk[e] = *reinterpret_cast<const uint32_t*>(&b);
      }
      out[u] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

void launch_q_prep(const QPrepArgs& a, cudaStream_t st) {
  if (a.T <= 0) return;
  if (a.v4 && a.q_head % 8 == 0 && a.q_head <= 1024 && a.nope % 8 == 0 && a.d_qk % 8 == 0 && a.rope % 2 == 0 &&
      a.nope + a.rope == a.q_head && (reinterpret_cast<uintptr_t>(a.q_full) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(a.q_eff) & 15) == 0) {
    launch_pdl(k_q_prep_v4_rows, dim3((unsigned)(((long long)a.T * a.H + 7) / 8)), dim3(256), 0, st, 1, a);
    return;
  }
  // (pair accesses need even offsets: q_head, nope, d_qk and rope are even in both presets)
  if (!a.v4 && a.q_head % 2 == 0 && a.nope % 2 == 0 && a.d_qk % 2 == 0 && a.rope % 2 == 0)
    launch_pdl(k_q_rope_token, dim3(a.T), dim3(256), 0, st, 1, a);
  else
    launch_pdl(k_q_prep, dim3(a.T * a.H), dim3(128), 0, st, 1, a);
}

// ---- split-KV attention on CUDA cores -----------------------------------------------------
// QK (reference src/fst_engine.cpp:3573-3589), softmax (3614-3666), SV (3668-3683) fused with
// an online softmax.  One block per schedule segment; 8 warps x 8 heads; 32-token tiles of
// the paged cache staged in shared memory; lane = cached token for QK, lane = column pair
// for SV.  Writes the un-normalised partial (max, sum, O).
constexpr int SIMT_TILE = 32;
constexpr int SIMT_HPW = 8;  // heads per warp

__global__ void __launch_bounds__(256, 1) k_attn_simt(AttnArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char smem[];
  const int stride = a.row * 2 + 16;  // bytes; the 16-byte pad keeps 16-byte loads conflict free
  bf16* s_q = reinterpret_cast<bf16*>(smem);  // [H, d_qk]
  unsigned char* s_tile = smem + (size_t)a.H * a.d_qk * 2;
  const AttnSeg seg = a.segs[blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* table = a.tables + seg.table;

  for (int h0 = 0; h0 < a.H; h0 += 8 * SIMT_HPW) {
    __syncthreads();
    {
      const uint4* src = reinterpret_cast<const uint4*>(a.q_eff + (long long)seg.tok * a.H * a.d_qk);
      uint4* dst = reinterpret_cast<uint4*>(s_q);
      for (int i = threadIdx.x; i < a.H * a.d_qk / 8; i += blockDim.x) dst[i] = src[i];
    }
    float m[SIMT_HPW], l[SIMT_HPW], acc[SIMT_HPW][16];
#pragma unroll
    for (int u = 0; u < SIMT_HPW; ++u) {
      m[u] = -INFINITY;
      l[u] = 0.0f;
#pragma unroll
      for (int c = 0; c < 16; ++c) acc[u][c] = 0.0f;
    }
    const int hbase = h0 + warp * SIMT_HPW;
    for (int s0 = seg.kv_begin; s0 < seg.kv_end; s0 += SIMT_TILE) {
      __syncthreads();
      const int per_row = a.row / 8;  // 16-byte pieces per cache row
      for (int i = threadIdx.x; i < SIMT_TILE * per_row; i += blockDim.x) {
        const int rr = i / per_row, cc = i % per_row;
        const int s = min(s0 + rr, seg.kv_end - 1);
        const long long prow = (long long)table[s / a.page_tokens] * a.page_tokens + s % a.page_tokens;
        *reinterpret_cast<uint4*>(s_tile + (size_t)rr * stride + cc * 16) =
            *reinterpret_cast<const uint4*>(a.pool + prow * a.row + cc * 8);
      }
      __syncthreads();
      // scores: lane = token of the tile
      float sc[SIMT_HPW];
#pragma unroll
      for (int u = 0; u < SIMT_HPW; ++u) sc[u] = 0.0f;
      const unsigned char* krow = s_tile + (size_t)lane * stride;
      for (int c = 0; c < a.d_qk / 8; ++c) {
        float kf[8];
        unpack8(*reinterpret_cast<const uint4*>(krow + c * 16), kf);
#pragma unroll
        for (int u = 0; u < SIMT_HPW; ++u) {
          if (hbase + u < a.H) {
            float qf[8];
            unpack8(*reinterpret_cast<const uint4*>(s_q + (size_t)(hbase + u) * a.d_qk + c * 8), qf);
#pragma unroll
            for (int e = 0; e < 8; ++e) sc[u] = fmaf(qf[e], kf[e], sc[u]);
          }
        }
      }
      const bool valid = s0 + lane < seg.kv_end;
      float p[SIMT_HPW];
#pragma unroll
      for (int u = 0; u < SIMT_HPW; ++u) {
        const float v = valid ? sc[u] * a.scale : -INFINITY;
        const float mn = fmaxf(m[u], warp_max(v));  // finite: every tile has a valid token
        const float alpha = expf(m[u] - mn);
        const float e = valid ? expf(v - mn) : 0.0f;
        l[u] = l[u] * alpha + warp_sum(e);
        m[u] = mn;
        p[u] = rbf(e);  // P is a bf16 operand of SV (reference 3651-3652)
#pragma unroll
        for (int c = 0; c < 16; ++c) acc[u][c] *= alpha;
      }
      // SV: lane owns columns lane*2 + 64*j (+1)
      const int ntok = min(SIMT_TILE, seg.kv_end - s0);
      for (int tk = 0; tk < ntok; ++tk) {
        float vf[16];
        const unsigned char* vrow = s_tile + (size_t)tk * stride;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j * 64 < a.d_v) {
            const float2 t2 = __bfloat1622float2(
                *reinterpret_cast<const __nv_bfloat162*>(vrow + (j * 64 + lane * 2) * 2));
            vf[2 * j] = t2.x;
            vf[2 * j + 1] = t2.y;
          } else {
            vf[2 * j] = vf[2 * j + 1] = 0.0f;
          }
        }
#pragma unroll
        for (int u = 0; u < SIMT_HPW; ++u) {
          const float pt = __shfl_sync(0xffffffffu, p[u], tk);
#pragma unroll
          for (int c = 0; c < 16; ++c) acc[u][c] = fmaf(pt, vf[c], acc[u][c]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < SIMT_HPW; ++u) {
      const int h = hbase + u;
      if (h < a.H) {
        if (lane == 0) {
          a.part_m[(long long)seg.part * a.H + h] = m[u];
          a.part_l[(long long)seg.part * a.H + h] = l[u];
        }
        float* o = a.part_o + ((long long)seg.part * a.H + h) * a.d_v;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j * 64 < a.d_v)
            *reinterpret_cast<float2*>(o + j * 64 + lane * 2) = make_float2(acc[u][2 * j], acc[u][2 * j + 1]);
      }
    }
  }
}

void launch_attn_simt(const AttnArgs& a, cudaStream_t st) {
  if (a.n_segs <= 0) return;
  const size_t smem = (size_t)a.H * a.d_qk * 2 + (size_t)SIMT_TILE * (a.row * 2 + 16);
  launch_pdl(k_attn_simt, dim3(a.n_segs), dim3(256), smem, st, 1, a);
}

// ---- log-sum-exp merge ---------------------------------------------------------------------
// out = sum_p e^{m_p - M} O_p / (sum_p e^{m_p - M} l_p [+ e^{sink - M}] + 1e-12); the sink and
// the 1e-12 guard are those of the reference softmax (src/fst_engine.cpp:3623, 3636, 3646).
// V4 applies the inverse RoPE of 3716 to the rounded output tail.
__device__ __forceinline__ void finish_row(float* s_out, bf16* o_row, const float* lut, int d_v,
                                           int rope, int inv_rope) {
  if (inv_rope) {
    __syncthreads();
    for (int p = threadIdx.x; p < rope / 2; p += blockDim.x) {
      const int j = d_v - rope + 2 * p;
      const float c = lut[2 * p], s = -lut[2 * p + 1], x0 = s_out[j], x1 = s_out[j + 1];
      s_out[j] = x0 * c - x1 * s;
      s_out[j + 1] = x0 * s + x1 * c;
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < d_v; j += blockDim.x) o_row[j] = f2bf(s_out[j]);
}

// One block per query row (token, head).  8 warps take the parts round-robin, a lane owns
// columns lane*4 + 128*j; the warps' sums are then added in warp order (deterministic).
constexpr int MERGE_THREADS = 256;  // rows with few parts use 128 threads, one per 4 columns

struct PartRef {
  float m, l;
  const float* o;
};

template <class GetPart>
__device__ __forceinline__ void merge_row(int n_parts, GetPart get, const float* sinks, int h, int d_v,
                                          float* s_acc /* [8][512] */, float* s_red /* [32] */, float& M_out,
                                          float& den_out) {
  if (blockDim.x == 128) {
    // few parts per row: every thread walks all parts for its own 4 columns, no exchange
    const bool sk = sinks != nullptr;
    float M = sk ? sinks[h] : -INFINITY;
    for (int p = 0; p < n_parts; ++p) M = fmaxf(M, get(p).m);
    float den = sk ? expf(sinks[h] - M) : 0.0f;
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
    const int col = threadIdx.x * 4;
    for (int p = 0; p < n_parts; ++p) {
      const PartRef pr = get(p);
      if (pr.m == -INFINITY) continue;
      const float w = expf(pr.m - M);
      den += w * pr.l;
      if (col < d_v) {
        const float2 v0 = *reinterpret_cast<const float2*>(pr.o + col);
        const float2 v1 = *reinterpret_cast<const float2*>(pr.o + col + 2);
        a4[0] = fmaf(w, v0.x, a4[0]);
        a4[1] = fmaf(w, v0.y, a4[1]);
        a4[2] = fmaf(w, v1.x, a4[2]);
        a4[3] = fmaf(w, v1.y, a4[3]);
      }
    }
    if (col < d_v) *reinterpret_cast<float4*>(s_acc + col) = make_float4(a4[0], a4[1], a4[2], a4[3]);
    __syncthreads();
    M_out = M;
    den_out = den;
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool sink = sinks != nullptr;
  // reference maximum over all parts (and the sink)
  float M = sink ? sinks[h] : -INFINITY;
  for (int p = threadIdx.x; p < n_parts; p += blockDim.x) M = fmaxf(M, get(p).m);
  M = warp_max(M);
  if (lane == 0) s_red[warp] = M;
  __syncthreads();
  M = s_red[0];
  for (int w = 1; w < nw; ++w) M = fmaxf(M, s_red[w]);
  __syncthreads();
  float acc[16];
#pragma unroll
  for (int c = 0; c < 16; ++c) acc[c] = 0.0f;
  float den = 0.0f;
  for (int p = warp; p < n_parts; p += nw) {
    const PartRef pr = get(p);
    if (pr.m == -INFINITY) continue;
    const float w = expf(pr.m - M);
    den += w * pr.l;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = lane * 4 + 128 * j;
      if (col < d_v) {
        // 8-byte loads: a gathered partial row starts 8 bytes into its (max, sum, O) record
        const float2 v0 = *reinterpret_cast<const float2*>(pr.o + col);
        const float2 v1 = *reinterpret_cast<const float2*>(pr.o + col + 2);
        acc[4 * j] = fmaf(w, v0.x, acc[4 * j]);
        acc[4 * j + 1] = fmaf(w, v0.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(w, v1.x, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(w, v1.y, acc[4 * j + 3]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int col = lane * 4 + 128 * j;
    if (col < d_v)
      *reinterpret_cast<float4*>(s_acc + warp * 512 + col) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
  }
  if (lane == 0) s_red[8 + warp] = den;
  __syncthreads();
  den = sink ? expf(sinks[h] - M) : 0.0f;
  for (int w = 0; w < nw; ++w) den += s_red[8 + w];
  // column sums over the warps, in warp order, left in s_acc[0][*]
  for (int col = threadIdx.x; col < d_v; col += blockDim.x) {
    float v = 0.0f;
    for (int w = 0; w < nw; ++w) v += s_acc[w * 512 + col];
    s_acc[col] = v;  // only this thread reads column `col` of the other warps' rows
  }
  __syncthreads();
  M_out = M;
  den_out = den;
}


__global__ void __launch_bounds__(MERGE_THREADS) k_merge(MergeArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float s_acc[8 * 512];
  __shared__ float s_red[32];
  const int r = blockIdx.x, t = r / a.H, h = r % a.H;
  const int p0 = a.tok_part[t], n_parts = a.tok_part[t + 1] - p0;
  if (a.skip_single && n_parts == 1) return;  // finished by the attention kernel
  auto get = [&](int p) {
    const long long i = (long long)(p0 + p) * a.H + h;
    return PartRef{a.part_m[i], a.part_l[i], a.part_o + i * a.d_v};
  };
  float M, den;
  merge_row(n_parts, get, a.sinks, h, a.d_v, s_acc, s_red, M, den);
  if (a.mode == 1) {
    float* o = a.rank_partial + (long long)r * (2 + a.d_v);
    if (threadIdx.x == 0) {
      o[0] = M;
      o[1] = den;
    }
    for (int j = threadIdx.x; j < a.d_v; j += blockDim.x) o[2 + j] = s_acc[j];
    return;
  }
  const float inv = den > 0.0f ? 1.0f / (den + 1e-12f) : 0.0f;
  for (int j = threadIdx.x; j < a.d_v; j += blockDim.x) s_acc[j] = rbf(s_acc[j] * inv);
  finish_row(s_acc, a.o_lat + (long long)r * a.d_v, a.lut + (long long)t * a.rope, a.d_v, a.rope, h < a.inv_rope);
}

// Rows with few parts: one WARP per query row (token, head), eight rows per block, nothing
// shared.  A lane owns columns lane*4 + 128*j and walks the parts in order, so the arithmetic per
// column is that of the 128-thread mode of merge_row.
__global__ void __launch_bounds__(256) k_merge_rows(MergeArgs a) {
  pdl_launch();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + warp;
  if (r < a.T * a.H) {
    const int t = r / a.H, h = r % a.H;
    const int p0 = a.tok_part[t], n_parts = a.tok_part[t + 1] - p0;
    if (a.skip_single && n_parts == 1) return;  // finished by the attention kernel
    const bool sk = a.sinks != nullptr;
    // Lane p holds (max, sum) of part p of a chunk of 32 parts: one round trip for the statistics of
    // all parts instead of one per part; the parts themselves are walked in order, as before.
    float M = sk ? a.sinks[h] : -INFINITY;
    float m_l = -INFINITY;
    for (int base = 0; base < n_parts; base += 32) {
      m_l = base + lane < n_parts ? a.part_m[(long long)(p0 + base + lane) * a.H + h] : -INFINITY;
      M = fmaxf(M, warp_max(m_l));
    }
    float den = sk ? expf(a.sinks[h] - M) : 0.0f;
    float acc[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.0f;
    for (int base = 0; base < n_parts; base += 32) {
      const bool mine = base + lane < n_parts;
      const long long i_l = (long long)(p0 + base + (mine ? lane : 0)) * a.H + h;
      if (n_parts > 32) m_l = mine ? a.part_m[i_l] : -INFINITY;  // (one chunk: still in the register)
      const float l_l = mine ? a.part_l[i_l] : 0.0f;
      const float w_l = m_l == -INFINITY ? 0.0f : expf(m_l - M);
      const int cnt = min(32, n_parts - base);
      for (int p = 0; p < cnt; ++p) {
        const long long i = (long long)(p0 + base + p) * a.H + h;
        const float m = __shfl_sync(0xffffffffu, m_l, p);
        const float w = __shfl_sync(0xffffffffu, w_l, p);
        const float lp = __shfl_sync(0xffffffffu, l_l, p);
        if (m == -INFINITY) continue;
        den += w * lp;
        const float* o = a.part_o + i * a.d_v;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = lane * 4 + 128 * j;
          if (col < a.d_v) {
            const float4 v = *reinterpret_cast<const float4*>(o + col);
            acc[4 * j] = fmaf(w, v.x, acc[4 * j]);
            acc[4 * j + 1] = fmaf(w, v.y, acc[4 * j + 1]);
            acc[4 * j + 2] = fmaf(w, v.z, acc[4 * j + 2]);
            acc[4 * j + 3] = fmaf(w, v.w, acc[4 * j + 3]);
          }
        }
      }
    }
    if (a.mode == 1) {
      float* o = a.rank_partial + (long long)r * (2 + a.d_v);
      if (lane == 0) {
        o[0] = M;
        o[1] = den;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = lane * 4 + 128 * j;
        if (col < a.d_v) {
#pragma unroll
          for (int e = 0; e < 4; ++e) o[2 + col + e] = acc[4 * j + e];
        }
      }
    } else {
      const float inv = den > 0.0f ? 1.0f / (den + 1e-12f) : 0.0f;
      const float* lut = a.lut + (long long)t * a.rope;
      bf16* o_row = a.o_lat + (long long)r * a.d_v;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = lane * 4 + 128 * j;
        if (col < a.d_v) {
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = rbf(acc[4 * j + e] * inv);
          if (h < a.inv_rope && col >= a.d_v - a.rope) {
            // inverse RoPE of the rounded output tail (reference src/fst_engine.cpp:3716)
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              const int pr = (col + e - (a.d_v - a.rope)) / 2;
              const float c = lut[2 * pr], s = -lut[2 * pr + 1], x0 = v[e], x1 = v[e + 1];
              v[e] = x0 * c - x1 * s;
              v[e + 1] = x0 * s + x1 * c;
            }
          }
          __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
          uint2 pk;
          pk.x = *reinterpret_cast<uint32_t*>(&lo);
          pk.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(o_row + col) = pk;
        }
      }
    }
  }
}

// Rows with MANY parts (one long sequence cut over all thread blocks): a block per (query row,
// group of 128 columns), so that the partials of a row are read by four blocks side by side; the
// eight warps of a block take the parts round-robin, a lane owns four columns, and the warps' sums
// are added in warp order (deterministic).
__global__ void __launch_bounds__(256) k_merge_wide(MergeArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float s_acc[8][128];
  __shared__ float s_red[16];
  const int r = blockIdx.x, cg = blockIdx.y, t = r / a.H, h = r % a.H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p0 = a.tok_part[t], n_parts = a.tok_part[t + 1] - p0;
  if (a.skip_single && n_parts == 1) return;
  const bool sk = a.sinks != nullptr;
  float M = sk ? a.sinks[h] : -INFINITY;
  for (int p = threadIdx.x; p < n_parts; p += blockDim.x) M = fmaxf(M, a.part_m[(long long)(p0 + p) * a.H + h]);
  M = warp_max(M);
  if (lane == 0) s_red[warp] = M;
  __syncthreads();
  M = s_red[0];
  for (int w = 1; w < 8; ++w) M = fmaxf(M, s_red[w]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.0f;
  const int col = cg * 128 + lane * 4;
  // four parts per round, all their loads issued before the first use (a warp's parts are few and
  // far apart in memory: the loop is bound by round trips, not by bytes)
  for (int pb = warp; pb < n_parts; pb += 32) {
    float m4[4], l4[4];
    float4 v4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int p = pb + 8 * q;
      const bool on = p < n_parts;
      const long long i = (long long)(p0 + (on ? p : pb)) * a.H + h;
      m4[q] = on ? a.part_m[i] : -INFINITY;
      l4[q] = a.part_l[i];
      v4[q] = *reinterpret_cast<const float4*>(a.part_o + i * a.d_v + col);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (m4[q] == -INFINITY) continue;
      const float w = expf(m4[q] - M);
      den += w * l4[q];
      acc.x = fmaf(w, v4[q].x, acc.x);
      acc.y = fmaf(w, v4[q].y, acc.y);
      acc.z = fmaf(w, v4[q].z, acc.z);
      acc.w = fmaf(w, v4[q].w, acc.w);
    }
  }
  *reinterpret_cast<float4*>(&s_acc[warp][lane * 4]) = acc;
  if (lane == 0) s_red[8 + warp] = den;
  __syncthreads();
  if (warp != 0) return;
  den = sk ? expf(a.sinks[h] - M) : 0.0f;
  for (int w = 0; w < 8; ++w) den += s_red[8 + w];
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  for (int w = 0; w < 8; ++w) {
    const float4 x = *reinterpret_cast<const float4*>(&s_acc[w][lane * 4]);
    v[0] += x.x;
    v[1] += x.y;
    v[2] += x.z;
    v[3] += x.w;
  }
  if (a.mode == 1) {
    float* o = a.rank_partial + (long long)r * (2 + a.d_v);
    if (cg == 0 && lane == 0) {
      o[0] = M;
      o[1] = den;
    }
    for (int e = 0; e < 4; ++e) o[2 + col + e] = v[e];
    return;
  }
  const float inv = den > 0.0f ? 1.0f / (den + 1e-12f) : 0.0f;
  for (int e = 0; e < 4; ++e) v[e] = rbf(v[e] * inv);
  if (h < a.inv_rope && col >= a.d_v - a.rope) {
    // inverse RoPE of the rounded output tail (reference src/fst_engine.cpp:3716)
    const float* lut = a.lut + (long long)t * a.rope;
    for (int e = 0; e < 4; e += 2) {
      const int pr = (col + e - (a.d_v - a.rope)) / 2;
      const float c = lut[2 * pr], sn = -lut[2 * pr + 1], x0 = v[e], x1 = v[e + 1];
      v[e] = x0 * c - x1 * sn;
      v[e + 1] = x0 * sn + x1 * c;
    }
  }
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  uint2 pk;
  pk.x = *reinterpret_cast<const uint32_t*>(&lo);
  pk.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(a.o_lat + (long long)r * a.d_v + col) = pk;
}

void launch_merge(const MergeArgs& a, cudaStream_t st) {
  if (a.T <= 0) return;
  if (a.threads != 128 && a.wide && a.d_v % 128 == 0 && a.rope % 4 == 0 && (a.d_v - a.rope) % 4 == 0) {
    launch_pdl(k_merge_wide, dim3(a.T * a.H, a.d_v / 128), dim3(256), 0, st, 1, a);
    return;
  }
  if (a.threads == 128 && a.d_v <= 512 && a.d_v % 4 == 0 && (a.rope % 2) == 0 && ((a.d_v - a.rope) % 4) == 0) {
    launch_pdl(k_merge_rows, dim3((a.T * a.H + 7) / 8), dim3(256), 0, st, 1, a);
    return;
  }
  launch_pdl(k_merge, dim3(a.T * a.H), dim3(a.threads == 128 ? 128 : MERGE_THREADS), 0, st, 1, a);
}

__global__ void __launch_bounds__(MERGE_THREADS) k_merge_gathered(MergeGatheredArgs a) {
  pdl_launch();
  pdl_wait();
  __shared__ __align__(16) float s_acc[8 * 512];
  __shared__ float s_red[32];
  const int r = blockIdx.x, t = r / a.H, h = r % a.H;
  const long long rows = (long long)a.T * a.H, w_row = 2 + a.d_v;
  auto get = [&](int p) {
    const float* pr = a.parts + (p * rows + r) * w_row;
    return PartRef{pr[0], pr[1], pr + 2};
  };
  float M, den;
  merge_row(a.n_parts, get, a.sinks, h, a.d_v, s_acc, s_red, M, den);
  const float inv = den > 0.0f ? 1.0f / (den + 1e-12f) : 0.0f;
  for (int j = threadIdx.x; j < a.d_v; j += blockDim.x) s_acc[j] = rbf(s_acc[j] * inv);
  finish_row(s_acc, a.o_lat + (long long)r * a.d_v, a.lut + (long long)t * a.rope, a.d_v, a.rope, h < a.inv_rope);
}

void launch_merge_gathered(const MergeGatheredArgs& a, cudaStream_t st) {
  if (a.T <= 0) return;
  launch_pdl(k_merge_gathered, dim3(a.T * a.H), dim3(a.n_parts <= 4 ? 128 : MERGE_THREADS), 0, st, 1, a);
}

// ---- V4 KV compressor ----------------------------------------------------------------------------
// The 127 non-negative E4M3 values, ascending (reference init_e4m3_grid, src/fst_engine.cpp:3070-3083).
__device__ __forceinline__ float e4m3_value(int i) {
  const int e = (i >> 3) & 15, m = i & 7;
  return e == 0 ? (float)m * 0.001953125f : ldexpf(1.0f + (float)m * 0.125f, e - 7);
}
// e4m3_roundtrip (3084-3100): the nearest grid value, ties to the even index.
__device__ __forceinline__ float e4m3_roundtrip(float v) {
  const float sign = v < 0.0f ? -1.0f : 1.0f;
  const float ax = fminf(fabsf(v), 448.0f);
  int lo = 0, hi = 126;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (e4m3_value(mid) <= ax) lo = mid; else hi = mid - 1;
  }
  int best = lo;
  if (best < 126) {
    const float bd = fabsf(ax - e4m3_value(best)), nd = fabsf(ax - e4m3_value(best + 1));
    if (nd < bd || (nd == bd && ((best + 1) & 1) == 0 && (best & 1) != 0)) ++best;
  }
  return sign * e4m3_value(best);
}

// One block per sequence of the call; thread j owns dim j of the pooled row (kv_lora <= 1024).
__global__ void __launch_bounds__(512) k_compress(CompressArgs a) {
  pdl_launch();
  pdl_wait();
  extern __shared__ float s_out[];  // [kv_lora]
  __shared__ float scratch[32];
  const CompressStep st = a.steps[blockIdx.x];
  const int ratio = a.ratio, width = a.width, hd = a.kv_lora;
  const int rows = ratio == 4 ? 8 : ratio;
  float* skv = a.state + (long long)st.slot * 2 * rows * width;
  float* ssc = skv + (long long)rows * width;
  for (int m = 0; m < st.q_len; ++m) {
    const int t = st.tok0 + m;
    const CompressTok tk = a.toks[t];
    const int pos_mod = tk.pos % ratio;
    const int row = ratio == 4 ? ratio + pos_mod : pos_mod;
    // state write: the value row, and the gate row with its positional bias (3194-3202)
    const bf16* pr = a.proj + (long long)t * 2 * width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
      skv[(long long)row * width + j] = bf2f(pr[j]);
      ssc[(long long)row * width + j] = bf2f(pr[width + j]) + a.ape[(long long)pos_mod * width + j];
    }
    __syncthreads();
    if (((tk.pos + 1) % ratio) != 0) continue;  // (uniform over the block)
    // per-dim softmax pool over the window rows, two lanes for ratio 4 (3206-3242)
    float pooled = 0.0f;
    const int j = threadIdx.x;
    if (j < hd) {
      float mx = -1e30f;
      for (int r = 0; r < ratio; ++r) {
        mx = fmaxf(mx, ssc[(long long)r * width + j]);
        if (ratio == 4) mx = fmaxf(mx, ssc[(long long)(ratio + r) * width + hd + j]);
      }
      if (mx > -0.5e30f) {
        float denom = 0.0f, sum = 0.0f;
        for (int r = 0; r < ratio; ++r) {
          const float wp = expf(ssc[(long long)r * width + j] - mx);
          if (ratio == 4) {
            const float wc = expf(ssc[(long long)(ratio + r) * width + hd + j] - mx);
            denom += wp + wc;
            sum += wp * skv[(long long)r * width + j];
            sum += wc * skv[(long long)(ratio + r) * width + hd + j];
          } else {
            denom += wp;
            sum += wp * skv[(long long)r * width + j];
          }
        }
        pooled = denom > 0.0f ? sum / denom : 0.0f;
      }
    }
    // RMS norm with the compressor's weight (3244-3250)
    const float ss = block_sum(pooled * pooled, scratch);
    const float rms = 1.0f / sqrtf(ss / (float)hd + 1e-6f);
    if (j < hd) s_out[j] = pooled * rms * bf2f(a.norm[j]);
    __syncthreads();
    // RoPE on the tail at the compressed position (3252-3254): interleaved pairs
    if (j < a.rope / 2) {
      const float* lut = a.lut + (long long)t * a.rope;
      const int k = hd - a.rope + 2 * j;
      const float c = lut[2 * j], s = lut[2 * j + 1], x0 = s_out[k], x1 = s_out[k + 1];
      s_out[k] = x0 * c - x1 * s;
      s_out[k + 1] = x0 * s + x1 * c;
    }
    __syncthreads();
    // E4M3 round trip of the nope part in blocks of 64 with a power-of-two scale (3256-3267)
    float v = 0.0f;
    if (j < hd) {
      v = s_out[j];
      if (j < hd - a.rope) {
        const int b0 = j & ~63;
        float amax = 0.0f;
        for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(s_out[b0 + i]));
        amax = fmaxf(amax, 1.0e-4f);
        const float scale = ldexpf(1.0f, (int)ceilf(log2f(amax / 448.0f)));
        v = e4m3_roundtrip(fminf(448.0f, fmaxf(-448.0f, v / scale))) * scale;
      }
      if (tk.dst >= 0) a.pool[tk.dst + j] = f2bf(v);
    }
    // window rotation, ratio 4 (3302-3317): the window just processed becomes the previous one
    if (ratio == 4) {
      for (int i = threadIdx.x; i < ratio * width; i += blockDim.x) {
        skv[i] = skv[(long long)ratio * width + i];
        ssc[i] = ssc[(long long)ratio * width + i];
      }
    }
    __syncthreads();
  }
}

void launch_compress(const CompressArgs& a, cudaStream_t st) {
  if (a.n_steps <= 0) return;
  launch_pdl(k_compress, dim3(a.n_steps), dim3(512), a.kv_lora * sizeof(float), st, 1, a);
}

// ---- bounded-wait self-test ----------------------------------------------------------------------
__global__ void k_wait_selftest(int* d_status, uint32_t polls) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
  }
  __syncthreads();
  // phase 0 never completes: nobody arrives.  Every thread's wait runs out (or sees the flag).
  tc::mbar_wait(&bar, 0, &abort_flag, d_status, ST_SELFTEST_TIMEOUT, polls);
}

void launch_wait_selftest(int* d_status, uint32_t polls, cudaStream_t st) {
  k_wait_selftest<<<1, 32, 0, st>>>(d_status, polls);
}

// Zero whole cache rows (speculative rollback, reference src/fst_engine.cpp:6132-6147).
__global__ void k_zero_rows(bf16* pool, const long long* row_off, int row) {
  bf16* p = pool + row_off[blockIdx.x];
  for (int j = threadIdx.x; j < row; j += blockDim.x) p[j] = f2bf(0.0f);
}

void launch_zero_rows(bf16* pool, const long long* row_off, int n_rows, int row, cudaStream_t st) {
  if (n_rows <= 0) return;
  k_zero_rows<<<n_rows, 128, 0, st>>>(pool, row_off, row);
}

}  // namespace fst
